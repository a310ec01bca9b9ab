"""A plain, slow Tugelorn: whole sequences, float64, no cache, no state carried between calls.

Nothing here is imported from the package.  One function per mechanism; ``forward`` strings them
together from a config.json dictionary and a dict of tensors by name.  Also the random weights and the
configurations of the tests.
"""
import math

import torch

F64 = torch.float64


# ---------------------------------------------------------------------------------------------
# mechanisms
# ---------------------------------------------------------------------------------------------
def rms_norm(x, w, eps):
    return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def rotate_pairs(x, positions, dims, base, factor):
    """x [T, heads, d]: coordinates (2i, 2i + 1), i < dims / 2, turned by positions * base^(-2i/dims) / factor."""
    i = torch.arange(dims // 2, dtype=F64)
    freq = torch.pow(torch.tensor(base, dtype=F64), -2.0 * i / dims) / factor
    ang = positions.to(F64)[:, None, None] * freq[None, None, :]
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = even * ang.cos() - odd * ang.sin()
    out[..., 1:dims:2] = odd * ang.cos() + even * ang.sin()
    return out


def query_temperature(positions, coef, every):
    return 1.0 + coef * torch.log(torch.div(positions + 1, every, rounding_mode="floor").to(F64) + 1.0)


def softmax_attention(q, k, v, scale, window):
    """q [T, H, d], k [T, G, d], v [T, G, dv] of one sequence from position 0; a query at i sees the keys
    max(0, i - window + 1) .. i (all of 0 .. i without a window)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    idx = torch.arange(T)
    seen = idx[None, :] <= idx[:, None]
    if window is not None:
        seen &= (idx[:, None] - idx[None, :]) < window
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def causal_conv_silu(x, taps_w):
    """x [T, C], taps_w [C, taps]: y_t = sum_j taps_w[:, j] x_{t - (taps - 1 - j)}, zeros before the start; silu."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x], dim=0)
    y = sum(padded[j:j + T] * taps_w[:, j] for j in range(taps))
    return y * torch.sigmoid(y)


def unit_rows(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + eps)


def delta_rule(q, k, v, beta, decay):
    """q, k, decay [T, H, dk], v [T, H, dv], beta [T, H] -> o [T, H, dv]; S [H, dk, dv] starts at zero."""
    T, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[2], dtype=F64)
    out = torch.zeros_like(v)
    for t in range(T):
        S = decay[t][:, :, None] * S
        read = torch.einsum("hkv,hk->hv", S, k[t])
        u = beta[t][:, None] * (v[t] - read)
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def clamped_glu(gate, up, limit, slope=1.702):
    g = torch.clamp(gate, max=limit)
    u = torch.clamp(up, min=-limit, max=limit)
    return g * torch.sigmoid(slope * g) * (u + 1.0)


# ---------------------------------------------------------------------------------------------
# mixers and the model
# ---------------------------------------------------------------------------------------------
def attention_mixer(x, W, p, m, kind, positions):
    T = x.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = x @ W[p + "q"].T, x @ W[p + "k"].T, x @ W[p + "v"].T
    if kind == "attention_2":
        q, k, v = q + W[p + "q.b"], k + W[p + "k.b"], v + W[p + "v.b"]
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv)
    if m.get("rot"):
        r = m["rot"]
        factor = r["scaling"]["factor"] if r.get("scaling") else 1.0
        q = rotate_pairs(q, positions, r["dims"], r["base"], factor)
        k = rotate_pairs(k, positions, r["dims"], r["base"], factor)
    if m.get("q_temp"):
        q = q * query_temperature(positions, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    window = m["mask"]["size"] if m.get("mask") else None
    o = softmax_attention(q, k, v, m["scale"], window)
    return o.reshape(T, H * dv) @ W[p + "o"].T


def channel_delta_mixer(x, W, p, m, eps):
    T = x.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rows(causal_conv_silu(x @ W[p + "q"].T, W[p + "q.conv"]).view(T, G, dk)) * dk ** -0.5
    k = unit_rows(causal_conv_silu(x @ W[p + "k"].T, W[p + "k.conv"]).view(T, G, dk))
    v = causal_conv_silu(x @ W[p + "v"].T, W[p + "v.conv"]).view(T, H, dv)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(x @ W[p + "b"].T)
    pre = ((x @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]).view(T, H, dk)
    decay = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None] * torch.nn.functional.softplus(pre))
    o = delta_rule(q, k, v, beta, decay)
    o = o * torch.rsqrt((o * o).mean(dim=-1, keepdim=True) + eps) * W[p + "norm"]
    o = o * torch.sigmoid((x @ W[p + "g1"].T) @ W[p + "g2"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ W[p + "o"].T


def run_order(cfg):
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, False) for i in range(n)]
    a, b = lp["start"], lp["stop"]
    order = [(i, False) for i in range(a)]
    for r in range(lp["times"]):
        order += [(i, r > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(cfg, weights, tokens, stream_after_runs=None):
    """Logits [T, vocab] of one sequence (float64)."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    positions = torch.arange(len(tokens))
    first = W["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    h = first.clone()
    for i, again in run_order(cfg):
        if again:
            h = h + first
        layer, p = cfg["layers"][i], f"l{i}."
        x = rms_norm(h, W[p + "norm1"], eps)
        if layer["type"] == "channel_delta":
            a = channel_delta_mixer(x, W, p + "mix.", layer["mixer"], eps)
        else:
            a = attention_mixer(x, W, p + "mix.", layer["mixer"], layer["type"], positions)
        h = h + mult * rms_norm(a, W[p + "norm1b"], eps)
        if layer["mlp"] is not None:
            x = rms_norm(h, W[p + "norm2"], eps)
            y = clamped_glu(x @ W[p + "mlp.gate"].T, x @ W[p + "mlp.up"].T, layer["mlp"]["limit"]) @ W[p + "mlp.down"].T
            h = h + mult * rms_norm(y, W[p + "norm2b"], eps)
        if stream_after_runs is not None:
            stream_after_runs.append(h.clone())
    return (rms_norm(h, W["final.norm"], eps) @ W["head"].T).to(torch.float32)


def greedy(cfg, weights, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, weights, toks)[-1].argmax()))
    return toks[len(prompt):]


# ---------------------------------------------------------------------------------------------
# tensors of a configuration and random weights
# ---------------------------------------------------------------------------------------------
def tensor_shapes(cfg, ranks):
    """name -> shape; ``ranks[i] = (a_rank, g_rank)`` for the channel_delta layers."""
    D, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out[p + "norm1"] = out[p + "norm1b"] = (D,)
        if layer["type"] == "channel_delta":
            ra, rg = ranks[i]
            out.update({p + "mix.q": (G * d, D), p + "mix.k": (G * d, D), p + "mix.v": (H * dv, D),
                        p + "mix.q.conv": (G * d, m["conv"]), p + "mix.k.conv": (G * d, m["conv"]),
                        p + "mix.v.conv": (H * dv, m["conv"]), p + "mix.b": (H, D), p + "mix.A_log": (H,),
                        p + "mix.dt_bias": (H * d,), p + "mix.a1": (ra, D), p + "mix.a2": (H * d, ra),
                        p + "mix.g1": (rg, D), p + "mix.g2": (H * dv, rg), p + "mix.norm": (dv,),
                        p + "mix.o": (D, H * dv)})
        else:
            out.update({p + "mix.q": (H * d, D), p + "mix.k": (G * d, D), p + "mix.v": (G * dv, D),
                        p + "mix.o": (D, H * dv)})
            if layer["type"] == "attention_2":
                out.update({p + "mix.q.b": (H * d,), p + "mix.k.b": (G * d,), p + "mix.v.b": (G * dv,)})
        if layer["mlp"] is not None:
            F = layer["mlp"]["ff"]
            out.update({p + "norm2": (D,), p + "norm2b": (D,), p + "mlp.gate": (F, D), p + "mlp.up": (F, D),
                        p + "mlp.down": (D, F)})
    return out


def random_weights(cfg, ranks, seed, sharp=1.0):
    """Weights large enough that every mechanism moves the logits, rounded to bfloat16 (returned as float32).
    ``sharp`` multiplies the query projections of the attention layers: the softmax then sits on few keys."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, ranks).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") else name
        if leaf.startswith("norm") or name == "final.norm" or leaf == "mix.norm":
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
        elif leaf.endswith(".conv"):
            t = 0.6 * torch.randn(shape, generator=gen)
        elif leaf.endswith(".b") and len(shape) == 1:
            t = 0.5 * torch.randn(shape, generator=gen)
        elif leaf == "mix.A_log":
            t = 0.7 * torch.randn(shape, generator=gen) - 0.5
        elif leaf == "mix.dt_bias":
            t = torch.randn(shape, generator=gen) - 1.0
        elif name == "embed":
            t = torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) * (1.5 / math.sqrt(shape[-1]))
            layer = cfg["layers"][int(name[1:name.index(".")])] if name.startswith("l") else None
            if layer is not None and leaf == "mix.q" and layer["type"] != "channel_delta":
                t = t * sharp
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


# ---------------------------------------------------------------------------------------------
# configurations of the tests: (config.json dictionary, ranks of the delta layers, cache page size)
# ---------------------------------------------------------------------------------------------
def _attn(heads, kv, dim, vdim, scale, window=None, rot=None, q_temp=None, kind="attention"):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if rot[2] is not None:
            m["rot"]["scaling"] = {"factor": rot[2]}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": kind, "mixer": m}


def _delta(heads, kv, dim, vdim, conv):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}


def _mlp(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _model(width, vocab, eps, mult, layers, loop=None):
    cfg = {"architecture": "Tugelorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
           "layers": [dict(l, mlp=mlp) for l, mlp in layers]}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


CONFIGS = {
    # a window of 24 over pages of 8, partial rotation (16 of 32 coordinates), the loop starts at layer 0,
    # value heads wider than key heads in the layer with biases
    "P": (_model(64, 211, 1e-5, 0.5, [
        (_attn(4, 2, 32, 32, 0.2, window=24, rot=(16, 10000.0, 2.0)), _mlp(96, 1.5)),
        (_delta(4, 2, 16, 32, 3), None),
        (_attn(2, 1, 32, 48, 0.15, q_temp=(0.5, 16), kind="attention_2"), _mlp(80, 3.0)),
    ], loop=(0, 2, 2)), {1: (8, 8)}, 8),
    # the delta layer first, a key size that is no multiple of 8, ranks that are none either, one q/k head
    # per value head, residual_mult 1, three passes over two layers, head size 64 (tensor-core kernels in
    # bfloat16) and a value size of 128 beside a key size of 64, rotation without scaling, a window of 70
    "Q": (_model(96, 300, 1e-6, 1.0, [
        (_delta(3, 3, 24, 40, 4), None),
        (_attn(4, 4, 64, 64, 0.13, q_temp=(0.25, 50), kind="attention_2"), _mlp(160, 2.5)),
        (_attn(4, 2, 64, 128, 0.11, window=70, rot=(64, 250000.0, None)), None),
        (_delta(4, 1, 32, 16, 2), _mlp(64, 1.0)),
    ], loop=(1, 3, 3)), {0: (6, 10), 3: (16, 4)}, 16),
    # no loop at all, a single head everywhere, a window of one page, a convolution of one tap
    "R": (_model(48, 130, 1e-4, 0.25, [
        (_attn(1, 1, 16, 16, 0.3, window=16, rot=(8, 100.0, 1.0)), _mlp(48, 2.0)),
        (_delta(1, 1, 8, 8, 1), _mlp(40, 2.0)),
        (_attn(1, 1, 16, 16, 0.25, q_temp=(1.0, 1), kind="attention_2"), None),
    ]), {1: (4, 4)}, 16),
    # sizes that are multiples of nothing: width 100, head sizes 20 / 12 and 10 / 6, three heads on one, five
    # taps, ranks 3 and 7, a window of 5, six rotated coordinates, the whole model looped twice
    "S": (_model(100, 257, 2e-5, 0.35, [
        (_attn(3, 1, 20, 12, 0.22, window=5, rot=(6, 3000.0, 1.5)), _mlp(150, 2.0)),
        (_delta(3, 1, 10, 6, 5), _mlp(90, 4.0)),
        (_attn(3, 3, 12, 20, 0.3, q_temp=(0.35, 3), kind="attention_2"), None),
    ], loop=(0, 3, 2)), {1: (3, 7)}, 4),
}


def config(name):
    """(config.json dictionary with the ranks written into the delta layers, ranks, page size)"""
    import copy
    cfg, ranks, page = CONFIGS[name]
    return copy.deepcopy(cfg), dict(ranks), page
