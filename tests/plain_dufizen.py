"""Plain implementation of Dufizen: whole sequences in float64, no cache, no state between calls, one function
per mechanism, nothing imported from the package.  The oracle of ``test_dufizen.py``.

Notation: x [T, D] the residual stream, h a sublayer's input, W[name] the tensors (linear weights [out, in]).
"""
import math

import torch

F64 = torch.float64


# ---------------------------------------------------------------------------------------------
# mechanisms
# ---------------------------------------------------------------------------------------------
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    """Plain weight."""
    return unit_rms(x, eps) * w


def zero_centred_norm(x, w, eps):
    """The model's norm: the stored weight lies around zero."""
    return unit_rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate(x, pos, base, dims):
    """x [T, ..., n]: pairs (i, i + dims / 2) of the first ``dims`` coordinates turn by pos * base^(-2i / dims)."""
    half = dims // 2
    if half == 0:
        return x
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = pos.to(F64)[:, None] * freq
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def gated_linear_recurrence(q, k, v, alpha, S0=None):
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t.  q, k, alpha [T, H, dk], v [T, H, dv]."""
    T, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[2], dtype=F64) if S0 is None else S0.clone()
    o = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def gla_mixer(h, W, p, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ W[p + "k"].T).view(T, H, dk)
    v = (h @ W[p + "v"].T).view(T, H, dv)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / m["tau"]).view(T, H, dk)
    o, _ = gated_linear_recurrence(q, k, v, alpha)
    o = rms_norm(o, W[p + "norm"], eps).reshape(T, H * dv)
    g = h @ W[p + "g"].T
    return (o * g * torch.sigmoid(g)) @ W[p + "o"].T


def sink_softmax(s, sink):
    """s [H, T, T] with -inf where a key is not seen; one more term exp(sink_h) in every denominator."""
    sink = sink.view(-1, 1, 1)
    mx = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - mx)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - mx))


def window_mask(T, size):
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    return (i - j >= 0) & (i - j < size)


def latent_attention_mixer(h, W, p, m, eps, use_sink=True):
    T = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    pos = torch.arange(T)
    q = (h @ W[p + "q"].T).view(T, H, d + r)
    low = h @ W[p + "dkv"].T
    c = rms_norm(low[:, :R], W[p + "dkv.norm"], eps)
    kr = rotate(low[:, R:], pos, base, dims)                 # one rotated key part for all heads
    qu, qr = q[..., :d], rotate(q[..., d:], pos, base, dims)
    ku = (c @ W[p + "uk"].T).view(T, H, d)
    v = (c @ W[p + "uv"].T).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", qu, ku) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    s = s.masked_fill(~window_mask(T, m["mask"]["size"]), -math.inf)
    sink = W[p + "sink"] if use_sink else torch.full((H,), -math.inf, dtype=F64)
    o = torch.einsum("hij,jhd->ihd", sink_softmax(s, sink), v)
    o = o * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "o"].T


def route(z, correction, r):
    """Router logits z [T, E] -> (indices [T, top], weights [T, top])."""
    E, top = r["experts"], r["top"]
    s = torch.softmax(z, -1)
    choice = s + correction
    if r.get("groups") is not None:
        G, keep = r["groups"]["count"], r["groups"]["keep"]
        best = choice.view(-1, G, E // G).max(-1).values.topk(keep, -1).indices
        ok = torch.zeros(z.shape[0], G, dtype=torch.bool).scatter_(1, best, True)
        choice = choice.masked_fill(~ok[:, :, None].expand(-1, G, E // G).reshape(-1, E), -math.inf)
    idx = choice.topk(top, -1).indices
    return idx, s.gather(1, idx)


def expert(h, up, down):
    return torch.relu(h @ up.T) ** 2 @ down.T


def moe(h, W, p, m):
    idx, w = route(h @ W[p + "router"].T, W[p + "correction"], m["router"])
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F64)
    for e in range(m["router"]["experts"]):
        rows, col = (idx == e).nonzero(as_tuple=True)
        if rows.numel():
            out[rows] += w[rows, col][:, None] * expert(h[rows], W[p + f"e{e}.up"], W[p + f"e{e}.down"])
    if m.get("shared") is not None:
        out = out + expert(h, W[p + "shared.up"], W[p + "shared.down"])
    return out


def token_side(x, tok, W, p, layer, dim, eps):
    e = W["side.embed"][tok][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ W[p + "side.gate"].T) * e) @ W[p + "side.proj"].T
    return rms_norm(y, W[p + "side.norm"], eps)


def run_order(cfg):
    """[(layer, pass or None)]."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if lp is None:
        return [(i, None) for i in range(n)]
    a, b, times = lp["start"], lp["stop"], lp["times"]
    return [(i, None) for i in range(a)] + [(i, t) for t in range(times) for i in range(a, b)] + \
           [(i, None) for i in range(b, n)]


def forward(cfg, W, tokens):
    """Logits [T, vocab] (float64) of one sequence."""
    W = {k: v.to(F64) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    tok = torch.tensor(tokens, dtype=torch.long)
    x = x0 = W["embed"][tok]
    side = cfg["token_side"]["dim"] if cfg.get("token_side") is not None else None
    for i, t in run_order(cfg):
        if t is not None and i == cfg["loop"]["start"]:
            x = torch.cat([x, x0], -1) @ W["loop.in"].T + W["loop.step"][t]
        L, p = cfg["layers"][i], f"l{i}."
        h = zero_centred_norm(x, W[p + "norm1"], eps)
        y = gla_mixer(h, W, p + "mix.", L["mixer"], eps) if L["type"] == "gla" else \
            latent_attention_mixer(h, W, p + "mix.", L["mixer"], eps)
        x = x + y * W[p + "ls1"]
        if L["mlp"] is not None:
            x = x + moe(zero_centred_norm(x, W[p + "norm2"], eps), W, p + "mlp.", L["mlp"]) * W[p + "ls2"]
        if side is not None:
            x = x + token_side(x, tok, W, p, i, side, eps)
    return zero_centred_norm(x, W["final.norm"], eps) @ W["embed"].T


def greedy(cfg, W, prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(forward(cfg, W, toks)[-1].argmax())
        out.append(t)
        toks.append(t)
    return out


# ---------------------------------------------------------------------------------------------
# configurations of the tests and random weights
# ---------------------------------------------------------------------------------------------
def latent(heads, dim, rot_dim, vdim, rank, window, scale, dims=None, base=10000.0):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim,
            "kv_rank": rank, "scale": scale, "mask": {"size": window},
            "rot": {"dims": rot_dim if dims is None else dims, "base": base}}}


def gla(heads, dim, vdim, tau):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}


def moe_cfg(experts, top, ff, groups=None, shared=None):
    r = {"experts": experts, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def model(vocab, width, eps, layers, loop=None, side=None):
    cfg = {"architecture": "Dufizen", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": [dict(mix, mlp=mlp) for mix, mlp in layers]}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if side is not None:
        cfg["token_side"] = {"dim": side}
    return cfg


# name -> (configuration, rank of the decay's narrow projection per layer, page size of the test)
CONFIGS = {
    # a loop from layer 0, two kinds of windows, groups of which one is kept, a side input
    "A": (model(96, 64, 1e-5,
                [(gla(2, 16, 24, 8.0), moe_cfg(8, 2, 32, groups=(2, 1), shared=48)),
                 (latent(3, 16, 8, 12, 32, 24, 0.2), moe_cfg(8, 2, 32, groups=(4, 3), shared=48)),
                 (gla(2, 16, 24, 8.0), None),
                 (latent(3, 16, 8, 12, 32, 17, 0.2), moe_cfg(8, 1, 32, groups=(2, 2)))],
                loop=(0, 2, 3), side=8), {0: 6, 2: 4}, 8),
    # sizes that are multiples of nothing: one head, a rotation of part of the rotated coordinates, no loop, no
    # side input, no shared expert, a layer without feed-forward
    "B": (model(77, 100, 1e-6,
                [(latent(1, 10, 6, 14, 20, 9, 0.3, dims=4, base=50.0), moe_cfg(6, 3, 20, groups=(3, 2))),
                 (gla(3, 12, 10, 2.5), None),
                 (latent(5, 6, 2, 6, 12, 30, 0.4, base=500.0), moe_cfg(5, 2, 12))]), {1: 5}, 4),
    # eight heads (a block of the attention kernel per token), larger heads, no groups, a loop in the middle
    "C": (model(200, 128, 1e-6,
                [(latent(8, 32, 16, 32, 64, 70, 0.15), moe_cfg(16, 4, 64, shared=64)),
                 (gla(4, 64, 64, 16.0), moe_cfg(16, 4, 64, groups=(4, 2), shared=64)),
                 (latent(2, 64, 32, 64, 128, 33, 0.1, dims=16), moe_cfg(4, 2, 128))],
                loop=(1, 2, 2), side=16), {1: 16}, 16),
    # twelve heads (a block's 16 rows are not all used), a latent size of six 16-column pairs, every layer looped,
    # every expert of a layer chosen, a tau below one
    "D": (model(300, 192, 1e-5,
                [(gla(5, 40, 56, 0.7), moe_cfg(12, 3, 48, groups=(3, 2), shared=80)),
                 (latent(12, 64, 32, 40, 96, 100, 0.12, base=3000.0), moe_cfg(4, 4, 16, groups=(2, 2)))],
                loop=(0, 2, 2), side=12), {0: 7}, 16),
    # two heads over a latent size of 256, a window shorter than a page, long keys in the recurrence
    "E": (model(150, 320, 1e-6,
                [(latent(2, 48, 64, 128, 256, 8, 0.2, dims=32), moe_cfg(8, 2, 40, shared=24)),
                 (gla(2, 128, 32, 30.0), moe_cfg(3, 1, 64))]), {1: 24}, 16),
}


def config(name):
    cfg, ranks, page = CONFIGS[name]
    return cfg, dict(ranks), page


def tensor_shapes(cfg, ranks):
    D, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, D), "final.norm": (D,)}
    if cfg.get("loop") is not None:
        s["loop.in"], s["loop.step"] = (D, 2 * D), (cfg["loop"]["times"], D)
    side = cfg["token_side"]["dim"] if cfg.get("token_side") is not None else None
    if side is not None:
        s["side.embed"] = (V, len(cfg["layers"]) * side)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"], s[p + "ls1"] = (D,), (D,)
        if L["type"] == "gla":
            qk, vw = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            s.update({p + "mix.q": (qk, D), p + "mix.k": (qk, D), p + "mix.v": (vw, D), p + "mix.g": (vw, D),
                      p + "mix.o": (D, vw), p + "mix.norm": (m["vdim"],), p + "mix.a1": (ranks[i], D),
                      p + "mix.a2": (qk, ranks[i]), p + "mix.a2.b": (qk,)})
        else:
            H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            s.update({p + "mix.q": (H * (d + r), D), p + "mix.dkv": (R + r, D), p + "mix.dkv.norm": (R,),
                      p + "mix.uk": (H * d, R), p + "mix.uv": (H * dv, R), p + "mix.sink": (H,), p + "mix.g": (H, D),
                      p + "mix.o": (D, H * dv)})
        if L["mlp"] is not None:
            q = L["mlp"]
            s[p + "norm2"], s[p + "ls2"] = (D,), (D,)
            s[p + "mlp.router"], s[p + "mlp.correction"] = (q["router"]["experts"], D), (q["router"]["experts"],)
            for e in range(q["router"]["experts"]):
                s[p + f"mlp.e{e}.up"], s[p + f"mlp.e{e}.down"] = (q["expert"]["ff"], D), (D, q["expert"]["ff"])
            if q.get("shared") is not None:
                s[p + "mlp.shared.up"], s[p + "mlp.shared.down"] = (q["shared"]["ff"], D), (D, q["shared"]["ff"])
        if side is not None:
            s.update({p + "side.gate": (side, D), p + "side.proj": (D, side), p + "side.norm": (D,)})
    return s


def random_weights(cfg, ranks, seed, sharp=1.0):
    """float32 tensors whose values are bfloat16 numbers.  Matrices ~ N(0, 1 / in); the query projections of the
    attention layers times ``sharp``; norm weights around zero, plain ones and layer scales around one; the decay's
    bias such that most of a state outlives a hundred tokens; sinks, corrections and side rows of visible size."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg, ranks).items():
        last = name.rsplit(".", 1)[-1]
        if len(shape) == 2 and name not in ("loop.step",):
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if name == "embed" or name == "side.embed":
                t = torch.randn(shape, generator=g)
            if name == "loop.in":
                t = t * math.sqrt(2.0)
        elif name == "loop.step":
            t = 0.5 * torch.randn(shape, generator=g)
        elif last in ("norm1", "norm2") or name == "final.norm":
            t = 0.2 * torch.randn(shape, generator=g)
        elif last in ("ls1", "ls2"):
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif last == "b":
            t = 4.0 + torch.randn(shape, generator=g)
        elif last == "sink":
            t = torch.randn(shape, generator=g)
        elif last == "correction":
            t = 0.1 * torch.randn(shape, generator=g) - 0.05     # choice scores of both signs
        else:   # plain norm weights
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        w[name] = t
    for i, L in enumerate(cfg["layers"]):
        if L["type"] == "latent_attention":
            w[f"l{i}.mix.q"] = w[f"l{i}.mix.q"] * sharp
            w[f"l{i}.mix.uk"] = w[f"l{i}.mix.uk"] * 2.0
        else:
            w[f"l{i}.mix.k"] = w[f"l{i}.mix.k"] * 0.5
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}
