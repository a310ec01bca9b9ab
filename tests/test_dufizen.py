"""Dufizen in the engine against the plain implementation of ``plain_dufizen``.

Configuration and plan on the CPU; on the GPU each kernel of the design alone, then whole models under every
way of cutting the work: whole prompts, token-by-token decoding from the first token, portions down to two
tokens, mixed batches with pages and state slots that are used again; keys just inside and just outside a
window, in prompts and in decoding; a far token that decides through the recurrent state; a sink that decides;
long decoding; greedy generation through the Python entry point and its scheduler; the programs.
"""
import copy
import json
import math
import os

import numpy as np
import pytest
import torch

import helpers
import plain_dufizen as plain

gpu = pytest.mark.gpu

TOL32 = 3e-5          # relative to the largest logit of the request
TOL16 = 6e-2
SHARP = {"float32": 3.0, "bfloat16": 1.5}   # the attention layers' queries times this: the softmax sits on few keys


def write_model(path, name=None, cfg=None, ranks=None, seed=0, sharp=1.0, edit=None):
    from safetensors.torch import save_file
    if cfg is None:
        cfg, ranks, _ = plain.config(name)
    w = plain.random_weights(cfg, ranks, seed, sharp)
    if edit is not None:
        edit(w)
        w = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}
    os.makedirs(path, exist_ok=True)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    return cfg, w


def engine_of(path, dtype, page, pool, max_requests=4, use_graphs=False, step_tokens=None):
    from ccinfer_b200.engine.engine import Engine, EngineOptions
    return Engine.from_model_dir(path, EngineOptions(
        dtype=dtype, page_size=page, kv_tokens=pool, max_requests=max_requests,
        max_tokens_per_step=step_tokens or pool, max_context=pool, use_graphs=use_graphs))


def compare(rows, ref, dtype, what):
    """32-bit: every row within TOL32.  bfloat16: a router picks its experts by a hard comparison, and rounding
    turns a close call the other way now and then, which moves that row by the size of an expert's output: up
    to one row in 25 may lie beyond TOL16 (seen: 1 in 45) while nine in ten lie within a third of it."""
    if dtype == "float32":
        return helpers.compare(rows, ref, TOL32, what)
    errs = []
    for (rid, pos), row in rows.items():
        assert np.isfinite(row).all(), what
        errs.append(float(np.abs(row - ref[rid][pos]).max()) / max(1e-6, float(np.abs(ref[rid]).max())))
    errs = np.sort(np.array(errs))
    beyond = int((errs > TOL16).sum())
    assert beyond <= max(1, len(errs) // 25), f"{what}: {beyond} of {len(errs)} rows beyond {TOL16}"
    p90 = errs[int(0.9 * (len(errs) - 1))]
    assert p90 <= TOL16 / 3, f"{what}: nine rows in ten should lie within {TOL16 / 3:.1e}, not {p90:.2e}"
    return float(p90)


def requests_of(cfg, lengths, seed):
    rng = np.random.RandomState(seed)
    return {f"r{i}": rng.randint(0, cfg["vocab"], size=n).tolist() for i, n in enumerate(lengths)}


# ---------------------------------------------------------------------------------------------
# CPU: configuration, plan
# ---------------------------------------------------------------------------------------------
def test_config_is_read_written_and_refused():
    from ccinfer_b200.config.dufizen import DufizenConfig
    from ccinfer_b200.config.registry import architecture_of
    from ccinfer_b200.errors import ModelConfigInvalid
    cfg, ranks, _ = plain.config("A")
    assert architecture_of(cfg).name == "Dufizen"
    c = DufizenConfig.from_json(cfg)
    assert c.loop == (0, 2, 3) and c.side_dim == 8 and c.layers[0].mixer.a_rank is None and c.layers[2].mlp is None
    assert c.layers[1].mixer.window == 24 and c.layers[3].mixer.window == 17 and c.layers[1].mixer.rot_dims == 8
    assert (c.layers[0].mlp.groups, c.layers[0].mlp.keep, c.layers[3].mlp.top, c.layers[3].mlp.shared_ff) == (2, 1, 1, 0)
    assert [i for i, _ in c.run_order()] == [0, 1, 0, 1, 0, 1, 2, 3]
    full = c.with_shapes(plain.tensor_shapes(cfg, ranks))
    assert (full.layers[0].mixer.a_rank, full.layers[2].mixer.a_rank) == (6, 4)
    assert DufizenConfig.from_json(full.to_json()) == full
    b = DufizenConfig.from_json(plain.config("B")[0])
    assert b.loop is None and b.side_dim is None and b.layers[0].mixer.rot_dims == 4 and b.layers[2].mlp.groups == 1
    with pytest.raises(ModelConfigInvalid):
        c.with_shapes({})
    for damage in (lambda j: j.pop("width"), lambda j: j["norm"].pop("eps"), lambda j: j["layers"][1]["mixer"].pop("scale"),
                   lambda j: j["layers"][1]["mixer"].pop("mask"), lambda j: j["layers"][1]["mixer"]["rot"].update(dims=10),
                   lambda j: j["layers"][0].update(type="attention"), lambda j: j["loop"].update(stop=9),
                   lambda j: j["layers"][0]["mixer"].pop("tau"), lambda j: j["layers"][0]["mlp"].update(kind="dense"),
                   lambda j: j["layers"][0]["mlp"]["router"].update(top=5),
                   lambda j: j["layers"][0]["mlp"]["router"]["groups"].update(count=3)):
        j = copy.deepcopy(cfg)
        damage(j)
        with pytest.raises(ModelConfigInvalid):
            DufizenConfig.from_json(j)


def test_plan_names_every_tensor_and_repeats_the_looped_layers():
    from ccinfer_b200.architectures.dufizen import build_plan
    from ccinfer_b200.config.dufizen import DufizenConfig
    for name in plain.CONFIGS:
        cfg, ranks, _ = plain.config(name)
        shapes = plain.tensor_shapes(cfg, ranks)
        plan = build_plan(DufizenConfig.from_json(cfg).with_shapes(shapes))
        plan.validate()
        assert {s.name: tuple(s.shape) for s in plan.tensor_specs()} == shapes
        start = cfg["loop"]["start"] if cfg.get("loop") else None
        want = [(i, t is not None and i == start, t if (t is not None and i == start) else 0)
                for i, t in plain.run_order(cfg)]
        assert [(e.layer, e.enter is not None, e.enter_number) for e in plan.order] == want
        assert plan.shared_tensor_names() >= {"embed"}


# ---------------------------------------------------------------------------------------------
# GPU: the kernels alone
# ---------------------------------------------------------------------------------------------
@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [48, 77, 1000])
def test_scaled_residual_kernel(dtype, D):
    from ccinfer_b200 import kernels
    g = torch.Generator().manual_seed(D)
    T = 5
    h, ls, w = torch.randn(T, D, generator=g), 1 + 0.3 * torch.randn(D, generator=g), 1 + 0.3 * torch.randn(D, generator=g)
    delta = (2 * torch.randn(T, D, generator=g)).to(dtype)
    want_h = h.double() + delta.double() * ls.double()
    tol = 1e-6 if dtype == torch.float32 else 8e-3
    for mode in ("norm", "rows", "sum"):
        hd = h.cuda()
        y = torch.empty(T, D, dtype=dtype, device="cuda") if mode != "sum" else None
        kernels.scaled_residual(hd, delta.cuda(), ls.cuda(), y=y, w_next=w.cuda() if mode == "norm" else None,
                                eps_next=1e-5)
        assert (hd.cpu().double() - want_h).abs().max() < 2e-6 * want_h.abs().max()
        if mode == "norm":
            want = plain.rms_norm(want_h, w.double(), 1e-5)
            assert (y.cpu().double() - want).abs().max() < tol * want.abs().max()
        elif mode == "rows":
            assert (y.cpu().double() - want_h).abs().max() < tol * want_h.abs().max()


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gelu_gate_rows_and_row_kernels(dtype):
    from ccinfer_b200 import kernels
    g = torch.Generator().manual_seed(3)
    T, n, V = 9, 10, 13
    z = (2 * torch.randn(T, 16, generator=g)).to(dtype)
    table = torch.randn(V, 40, generator=g).to(dtype)
    ids = torch.randint(0, V, (T,), generator=g).to(torch.int32)
    pending = torch.tensor([5, 7], dtype=torch.int32)
    ids[2] = -2                                   # the token last drawn for slot 1
    real = ids.clone().long()
    real[2] = 7
    want = plain.gelu_tanh(z[:, :n].double()) * table.double()[real][:, 20:20 + n]
    zd = z.cuda()
    kernels.gelu_gate_rows(zd[:, :n], table.cuda(), 20, ids.cuda(), pending=pending.cuda())
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    assert (zd[:, :n].cpu().double() - want).abs().max() < tol * want.abs().max()
    assert torch.equal(zd[:, n:].cpu(), z[:, n:])
    a, b = torch.randn(T, 6, generator=g), torch.randn(T, 6, generator=g)
    out = torch.empty(T, 12, dtype=dtype, device="cuda")
    kernels.concat_cast(out, a.cuda(), b.cuda())
    assert torch.equal(out.cpu(), torch.cat([a, b], 1).to(dtype))
    row = torch.randn(6, generator=g)
    ad = a.cuda()
    kernels.add_row(ad, row.cuda())
    assert torch.equal(ad.cpu(), a + row)


@gpu
@pytest.mark.parametrize("E,groups,keep,top", [(16, 4, 3, 4), (8, 2, 1, 2), (6, 3, 2, 3), (5, 1, 1, 2), (64, 8, 4, 8),
                                               (12, 4, 4, 1), (3, 1, 1, 3)])
def test_router_kernel(E, groups, keep, top):
    """Choice scores of both signs (a group that is not kept counts as minus infinity, not as zero), weights
    without the correction and not renormalised."""
    from ccinfer_b200 import kernels
    g = torch.Generator().manual_seed(E * 100 + top)
    T = 50
    z = 2 * torch.randn(T, E, generator=g)
    corr = 0.2 * torch.randn(E, generator=g) - 0.15
    r = {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}}
    idx, w = plain.route(z.double(), corr.double(), r)
    di = torch.empty(T, top, dtype=torch.int32, device="cuda")
    dw = torch.empty(T, top, device="cuda")
    dense = torch.empty(T, E, device="cuda")
    kernels.moe_route(z.cuda(), corr.cuda(), di, dw, dense, groups, keep)
    assert torch.equal(di.cpu().long(), idx)
    assert (dw.cpu().double() - w).abs().max() < 1e-6
    want = torch.zeros(T, E, dtype=torch.float64).scatter_(1, idx, w)
    assert (dense.cpu().double() - want).abs().max() < 1e-6
    assert top == E or (w.sum(-1) < 0.999).any()  # the weights are not renormalised


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sparse", [False, True])
@pytest.mark.parametrize("E,top,F,D,groups,SF", [(8, 2, 64, 64, (4, 2), 32), (16, 4, 32, 128, None, 0), (5, 5, 8, 40, None, 8),
                                                 (4, 2, 6, 22, (2, 1), 10)])
def test_mixture_of_experts_alone(dtype, sparse, E, top, F, D, groups, SF):
    """The part by itself, in both of its forms, from one token to so many that an expert's rows fill several
    tiles of every size."""
    from ccinfer_b200.engine.runtime import Runtime
    from ccinfer_b200.parts import MixtureOfExperts
    rt = Runtime("cuda:0", dtype, 640, 4)
    m = plain.moe_cfg(E, top, F, groups=groups, shared=SF or None)
    g = torch.Generator().manual_seed(E + F)
    W = {"router": 3 * torch.randn(E, D, generator=g) / math.sqrt(D), "correction": 0.1 * torch.randn(E, generator=g) - 0.05}
    for e in range(E):
        W[f"e{e}.up"] = torch.randn(F, D, generator=g) / math.sqrt(D)
        W[f"e{e}.down"] = torch.randn(D, F, generator=g) / math.sqrt(F)
    if SF:
        W["shared.up"], W["shared.down"] = torch.randn(SF, D, generator=g) / math.sqrt(D), torch.randn(D, SF, generator=g) / math.sqrt(SF)
    W = {k: v.to(torch.bfloat16).float() for k, v in W.items()}
    names = {"router": "router", "correction": "correction", "up": "e{e}.up", "down": "e{e}.down",
             "shared_up": "shared.up", "shared_down": "shared.down"}
    part = MixtureOfExperts(D, E, top, F, names, *(groups or (1, 1)), SF, sparse=sparse)
    part.bind(rt, lambda n: W[n].cuda().to(dtype) if W[n].dim() == 2 else W[n].cuda())
    # (the grouped products of the bfloat16 path want 16-byte rows; other sizes run the dense form)
    assert part.use_sparse == (sparse and (dtype == torch.float32 or (D % 8 == 0 and F % 8 == 0)))
    for T in (1, 5, 70, 300, 640):
        x = torch.randn(T, D, generator=g).to(torch.bfloat16)
        want = plain.moe(x.double(), {k: v.double() for k, v in W.items()}, "", m)
        got = part.forward(x.cuda().to(dtype), None).double().cpu()
        err = (got - want).abs().amax(-1) / want.abs().max()
        tol = 2e-6 if dtype == torch.float32 else 1.5e-2
        # (in bfloat16 a router's close call may go the other way for a token or two)
        assert (err > tol).sum() <= (0 if dtype == torch.float32 else max(1, T // 50)), (T, err.max())
    rt.check_status()


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batched_products(dtype):
    """A product per head over strided views (rows and heads at strides that are multiples of nothing)."""
    from ccinfer_b200.engine.runtime import Runtime
    rt = Runtime("cuda:0", dtype, 64, 4)
    g = torch.Generator().manual_seed(1)
    T, H, K, N = 21, 3, 10, 14
    x = torch.randn(T, H, K + 5, generator=g).to(dtype).cuda()
    w = torch.randn(H, N, K, generator=g).to(dtype).cuda()
    for out_dtype in (dtype, torch.float32):
        out = torch.zeros(T, H, N + 3, dtype=out_dtype, device="cuda")
        rt.linear_batched(out[:, :, :N].permute(1, 0, 2), x[:, :, :K].permute(1, 0, 2), w)
        want = torch.einsum("thk,hnk->thn", x[:, :, :K].double(), w.double())
        tol = 1e-6 if dtype == torch.float32 else (1e-2 if out_dtype == torch.bfloat16 else 1e-6)
        assert (out[:, :, :N].double() - want).abs().max() < tol * want.abs().max()
        assert (out[:, :, N:] == 0).all()


@gpu
@pytest.mark.parametrize("dk,dv,H", [(16, 24, 2), (12, 10, 3), (64, 64, 4), (130, 20, 1)])
def test_gated_linear_recurrence_kernels(dk, dv, H):
    """The recurrence over three launches (the state carried in between), two requests of unequal length, with a
    slot that is not in the step left alone; decays from tiny to one."""
    from ccinfer_b200 import kernels
    g = torch.Generator().manual_seed(dk)
    lens = [[5, 1], [1, 7], [20, 1]]
    total = [sum(x[i] for x in lens) for i in range(2)]
    proj = [torch.randn(n, 2 * H * dk + H * dv, generator=g).to(torch.bfloat16) for n in total]
    a = [(3 * torch.randn(n, H * dk, generator=g)).to(torch.bfloat16) for n in total]
    bias = 2 + torch.randn(H * dk, generator=g)
    tau = 3.0
    want = []
    for p, z in zip(proj, a):
        n = p.shape[0]
        pd = p.double()
        q = pd[:, :H * dk].view(n, H, dk) * dk ** -0.5
        k = pd[:, H * dk:2 * H * dk].view(n, H, dk)
        v = pd[:, 2 * H * dk:].view(n, H, dv)
        alpha = torch.sigmoid(z.double() + bias.double()).pow(1 / tau).view(n, H, dk)
        want.append(plain.gated_linear_recurrence(q, k, v, alpha))
    state = torch.zeros(4, H, dv, dk, device="cuda")
    state[1] = 7.0                                  # a slot of nobody's
    slots = torch.tensor([2, 0], dtype=torch.int32, device="cuda")
    at = [0, 0]
    for step in lens:
        rows = torch.cat([proj[i][at[i]:at[i] + step[i]] for i in range(2)]).cuda()
        arow = torch.cat([a[i][at[i]:at[i] + step[i]] for i in range(2)]).cuda()
        T = rows.shape[0]
        cu = torch.tensor([0, step[0], T], dtype=torch.int32, device="cuda")
        qn, kn, gg = (torch.empty(T, H, dk, device="cuda") for _ in range(3))
        vv, o = torch.empty(T, H, dv, device="cuda"), torch.empty(T, H, dv, device="cuda")
        kernels.gla_prepare(rows, (0, H * dk, 2 * H * dk), arow, bias.cuda(), qn, kn, vv, gg, H, dk, dv, dk ** -0.5, tau)
        kernels.gated_linear_recurrence(qn, kn, vv, gg, state, o, cu, slots, 2, H, dk, dv)
        for i, r0 in ((0, 0), (1, step[0])):
            ref = want[i][0][at[i]:at[i] + step[i]]
            assert (o[r0:r0 + step[i]].cpu().double() - ref).abs().max() < 2e-5 * max(1.0, ref.abs().max())
            at[i] += step[i]
    for i, s in ((0, 2), (1, 0)):
        ref = want[i][1].transpose(1, 2)            # the kernel keeps a column of S contiguous
        assert (state[s].cpu().double() - ref).abs().max() < 2e-5 * max(1.0, ref.abs().max())
    assert (state[1] == 7.0).all() and (state[3] == 0).all()


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,r,dims,dv,R,window,page", [(3, 16, 8, 8, 12, 32, 24, 8), (1, 10, 6, 4, 14, 20, 9, 4),
                                                         (8, 32, 16, 16, 32, 64, 70, 16), (2, 8, 4, 4, 8, 40, 1, 4),
                                                         (11, 4, 2, 2, 4, 12, 300, 16),
                                                         # sizes that the tensor-core form takes in bfloat16
                                                         (3, 16, 16, 16, 12, 32, 24, 8), (20, 8, 16, 8, 8, 48, 300, 8),
                                                         (1, 16, 32, 32, 16, 512, 40, 16),
                                                         (16, 16, 16, 16, 16, 128, 100, 16)])
def test_latent_attention_mixer_alone(dtype, H, d, r, dims, dv, R, window, page, tmp_path):
    """One layer of latent attention as a whole model would hide it behind other layers, so the mixer runs in a
    step of its own: a prompt, then portions and single tokens from the cache, against the plain mixer."""
    from ccinfer_b200.engine.engine import Engine, EngineOptions, StepEntry
    from ccinfer_b200.engine.plan import ModelPlan, RunEntry
    from ccinfer_b200.parts import LatentAttention, LayerScaleBlock, OutputHead, RMSNorm, TokenEmbedding
    D, V, eps, scale = 40, 30, 1e-5, 0.35
    g = torch.Generator().manual_seed(H * 7 + R)
    m = {"heads": H, "dim": d, "rot_dim": r, "vdim": dv, "kv_rank": R, "scale": scale, "mask": {"size": window},
         "rot": {"dims": dims, "base": 100.0}}
    shapes = {"q": (H * (d + r), D), "dkv": (R + r, D), "dkv.norm": (R,), "uk": (H * d, R), "uv": (H * dv, R),
              "sink": (H,), "g": (H, D), "o": (D, H * dv)}
    W = {"mix." + k: (torch.randn(s, generator=g) * (2.0 / math.sqrt(s[-1]) if len(s) == 2 else 1.0)) for k, s in shapes.items()}
    W["mix.dkv.norm"] = 1 + 0.2 * W["mix.dkv.norm"]
    W = {k: v.to(torch.bfloat16).float() for k, v in W.items()}
    names = {k.replace(".", "_"): "mix." + k for k in shapes}
    mixer = LatentAttention(D, H, d, r, dv, R, window, scale, 100.0, dims, eps, names)
    extra = {"embed": torch.randn(V, D, generator=g).to(torch.bfloat16).float(), "n": torch.zeros(D), "ls": torch.ones(D)}
    block = LayerScaleBlock(D, RMSNorm(D, eps, "n", weight_offset=1.0), mixer, ("ls", "ls2"))
    plan = ModelPlan(TokenEmbedding(V, D, "embed"), [block], [RunEntry(0)], RMSNorm(D, eps, "n", weight_offset=1.0),
                     OutputHead(D, V, "embed"), V)
    every = dict(W, **extra)
    dt = {torch.float32: "float32", torch.bfloat16: "bfloat16"}[dtype]

    def fetch(name):
        t = every[name].cuda()
        return t.to(dtype) if t.dim() == 2 else t

    eng = Engine(plan, fetch, EngineOptions(dtype=dt, page_size=page, kv_tokens=512, max_requests=3,
                                            max_tokens_per_step=512, max_context=512, use_graphs=False))
    rng = np.random.RandomState(0)
    toks = {"a": rng.randint(0, V, size=150).tolist(), "b": rng.randint(0, V, size=41).tolist()}
    want = {}
    for rid, t in toks.items():
        x = extra["embed"].double()[t]
        h = plain.unit_rms(x, eps)
        y = x + plain.latent_attention_mixer(h, {k: v.double() for k, v in W.items()}, "mix.", m, eps)
        want[rid] = (plain.unit_rms(y, eps) @ extra["embed"].double().T).numpy()
    steps = helpers.trace_mixed(toks, max_live=2, seed=2, portion_choices=(2, 3, 33, 9, 70))
    rows = helpers.replay(eng, steps)
    helpers.compare(rows, want, 2e-5 if dtype == torch.float32 else 5e-2, f"latent attention alone {dt}")


# ---------------------------------------------------------------------------------------------
# GPU: whole models under every cutting
# ---------------------------------------------------------------------------------------------
# prompt lengths just below, at and just above the windows (24, 17; 9, 30; 70, 33; 100; 8) and the pages' borders
LENGTHS = {"A": [1, 2, 16, 17, 18, 23, 24, 25, 26, 60, 97], "B": [1, 3, 8, 9, 10, 11, 29, 30, 31, 32, 75],
           "C": [2, 32, 33, 34, 35, 69, 70, 71, 72, 150], "D": [1, 15, 16, 17, 99, 100, 101, 102, 130],
           "E": [1, 7, 8, 9, 10, 16, 17, 40, 90]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name in plain.CONFIGS:
        for dtype, sharp in SHARP.items():
            d = str(tmp_path_factory.mktemp("duf" + name))
            cfg, w = write_model(d, name, seed=ord(name), sharp=sharp)
            reqs = requests_of(cfg, LENGTHS[name], 2)
            ref = {rid: plain.forward(cfg, w, t).numpy() for rid, t in reqs.items()}
            out[name, dtype] = (d, cfg, w, reqs, ref, plain.CONFIGS[name][2])
    return out


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(plain.CONFIGS))
@pytest.mark.parametrize("mode", ["whole", "decode from the first token", "decode40", "portions", "mixed"])
def test_replay_matches_plain(models, name, dtype, mode):
    d, cfg, w, reqs, ref, page = models[name, dtype]
    if mode == "whole":
        steps = helpers.trace_whole(reqs)
    elif mode == "decode from the first token":
        steps = helpers.trace_prefill_then_decode(reqs, tail=10 ** 6)
    elif mode == "decode40":
        steps = helpers.trace_prefill_then_decode(reqs, tail=40)
    elif mode == "portions":
        steps = helpers.trace_portions(reqs)
    else:
        steps = helpers.trace_mixed(reqs, max_live=4, seed=5)
    pool = helpers.max_live_tokens(steps, round_to=max(64, page))
    eng = engine_of(d, dtype, page, pool, max_requests=4)
    rows = helpers.replay(eng, steps)
    assert len(rows) == sum(len(t) for t in reqs.values())
    worst = compare(rows, ref, dtype, f"{name} {dtype} {mode}")
    print(f"[worst] {name}, {dtype}, {mode}: {worst:.3e}")
    eng.cache.check_consistency()
    assert all(p.used_pages == 0 for p in eng.cache.pools)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(plain.CONFIGS))
def test_replay_with_the_sparse_experts(models, name, dtype, monkeypatch):
    """The same models with the form of the mixture that runs only the chosen experts (which by itself starts at
    sizes far above these), mixed batches and graphs."""
    from ccinfer_b200.parts import MixtureOfExperts
    monkeypatch.setattr(MixtureOfExperts, "SPARSE_MIN_WEIGHTS", 0)
    calls = []
    inner = MixtureOfExperts._forward_sparse
    monkeypatch.setattr(MixtureOfExperts, "_forward_sparse", lambda self, x, T: (calls.append(T), inner(self, x, T))[1])
    d, cfg, w, reqs, ref, page = models[name, dtype]
    for steps, graphs in ((helpers.trace_whole(reqs), False), (helpers.trace_mixed(reqs, max_live=4, seed=7), True)):
        pool = helpers.max_live_tokens(steps, round_to=max(64, page))
        eng = engine_of(d, dtype, page, pool, max_requests=4, use_graphs=graphs)
        rows = helpers.replay(eng, steps)
        compare(rows, ref, dtype, f"{name} {dtype} sparse experts")
    assert calls or (name == "B" and dtype == "bfloat16")   # (rows of 100 bfloat16 values are no 16-byte rows)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_and_graphs(models, dtype):
    """Portions of more than 64 tokens after a cached prefix beside decode steps replayed from CUDA graphs."""
    d, cfg, w, reqs, ref, page = models["C", dtype]
    steps = helpers.trace_mixed(reqs, max_live=3, seed=13, prefill_frac=0.8, portion_choices=(70, 130, 65, 2, 100))
    pool = helpers.max_live_tokens(steps, round_to=64)
    eng = engine_of(d, dtype, page, pool, max_requests=4, use_graphs=True)
    rows = helpers.replay(eng, steps)
    worst = compare(rows, ref, dtype, f"C {dtype} long portions, graphs")
    print(f"[worst] C, {dtype}, long portions, graphs: {worst:.3e}")
    assert eng.graph_replays > 0


@gpu
def test_a_slot_that_is_used_again_starts_from_zero(models):
    """Two state slots, five requests one after another and in pairs: every later request gets a slot whose
    recurrent state an earlier one left behind."""
    d, cfg, w, reqs, ref, page = models["A", "float32"]
    eng = engine_of(d, "float32", page, 256, max_requests=2)
    ids = list(reqs)[5:10]
    for group in ([ids[0]], [ids[1], ids[2]], [ids[3], ids[4]]):
        steps = helpers.trace_mixed({r: reqs[r] for r in group}, max_live=2, seed=1)
        rows = helpers.replay(eng, steps)
        helpers.compare(rows, ref, TOL32, "slots used again")
    assert eng.cache.slots.free_slots == 2


def _one_layer(mix, side=None):
    return plain.model(64, 32, 1e-5, [(mix, None)], side=side)


@gpu
def test_a_key_at_the_windows_edge_decides(tmp_path):
    """One layer of latent attention with a window of 20.  Scores come from the shared key part alone, through
    two of its coordinates that do not turn, and read the first half of the stream; the latent vector (hence the
    values) reads the second half.  Tokens 0 and 1 share their first half and have opposite second halves, so the
    query of token 1 matches the key of token 0 as well as its own and hardly any other.  Token 1 ends the
    sequence; token 0 stands 19 places back (the last key the window keeps) or 20 places back (the first it
    drops): in one case the far token's value cancels the token's own, in the other it must not be seen.  In a
    prompt, in portions that end at the edge, and decoded."""
    cfg = _one_layer(plain.latent(2, 8, 4, 8, 16, 20, 1.0, dims=2))
    d = str(tmp_path / "edge")

    def edit(w):
        R, H, dq, r = 16, 2, 8, 4
        w["l0.norm1"] = torch.zeros_like(w["l0.norm1"])
        dkv = w["l0.mix.dkv"]
        dkv[:R, :16] = 0                   # the latent vector reads the second half of the stream
        dkv[R:R + 2] = 0                   # the pair that turns is not used
        dkv[R + 2:, 16:] = 0               # the key part reads the first half
        q = w["l0.mix.q"].view(H, dq + r, 32)
        q[:, :dq + 2] = 0
        q[:, dq + 2:] = dkv[R + 2:] * 30.0
        w["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], -3.0)
        w["embed"][2:, :16] *= 0.2
        w["embed"][1, :16] = w["embed"][0, :16]
        w["embed"][1, 16:] = -w["embed"][0, 16:]

    cfg, w = write_model(d, cfg=cfg, ranks={}, seed=11, edit=edit)
    rng = np.random.RandomState(0)
    for back in (19, 20):
        toks = rng.randint(2, 64, size=90).tolist()
        toks[-1 - back], toks[-1] = 0, 1
        ref = plain.forward(cfg, w, toks).numpy()
        other = list(toks)
        other[-1 - back] = 2
        moved = np.abs(ref[-1] - plain.forward(cfg, w, other).numpy()[-1]).max() / np.abs(ref[-1]).max()
        assert (moved > 0.1) == (back == 19), (back, moved)    # inside the window the key decides, outside it is gone
        for dtype in ("float32", "bfloat16"):
            eng = engine_of(d, dtype, 8, 128)
            reqs = {"a": toks}
            for steps in (helpers.trace_whole(reqs), helpers.trace_prefill_then_decode(reqs, tail=30),
                          helpers.trace_portions(reqs, sizes=(90 - back - 1, 2, back - 2, 1)),
                          helpers.trace_portions(reqs, sizes=(90 - back, back - 1, 1))):
                rows = helpers.replay(eng, steps)
                helpers.compare(rows, {"a": ref}, TOL32 if dtype == "float32" else TOL16, f"key {back} back")


@gpu
def test_a_sink_decides(tmp_path):
    """Sinks far above every score: most of each softmax's weight goes to the term that has no value.  Leaving it
    out would change the logits by their own size."""
    cfg = _one_layer(plain.latent(3, 8, 4, 8, 16, 12, 0.3))
    d = str(tmp_path / "sink")

    def edit(w):
        w["l0.mix.sink"] = torch.tensor([4.0, 6.0, -1.0])

    cfg, w = write_model(d, cfg=cfg, ranks={}, seed=12, edit=edit)
    toks = np.random.RandomState(1).randint(0, 64, size=40).tolist()
    ref = plain.forward(cfg, w, toks).numpy()
    W64 = {k: v.double() for k, v in w.items()}
    x = W64["embed"][toks]
    h = plain.zero_centred_norm(x, W64["l0.norm1"], 1e-5)
    a = plain.latent_attention_mixer(h, W64, "l0.mix.", cfg["layers"][0]["mixer"], 1e-5)
    b = plain.latent_attention_mixer(h, W64, "l0.mix.", cfg["layers"][0]["mixer"], 1e-5, use_sink=False)
    assert (a - b).abs().max() > 0.5 * b.abs().max()
    for dtype in ("float32", "bfloat16"):
        eng = engine_of(d, dtype, 4, 64)
        for steps in (helpers.trace_whole({"a": toks}), helpers.trace_prefill_then_decode({"a": toks}, tail=20)):
            rows = helpers.replay(eng, steps)
            helpers.compare(rows, {"a": ref}, TOL32 if dtype == "float32" else TOL16, "sink")


@gpu
def test_a_far_token_decides_through_the_state(tmp_path):
    """One layer of gated linear attention whose decay is nearly one.  Queries and keys read the first half of the
    stream, values the second; tokens 0 and 1 share their first half.  Token 0 stands at ONE far place among 400
    and token 1 at the end: what the state kept of the far token decides the last logits.  The far place is the
    first token, around a page border and the middle; the prompt is cut so that the state crosses steps."""
    cfg = _one_layer(plain.gla(2, 16, 16, 4.0))
    d = str(tmp_path / "far")

    def edit(w):
        w["l0.norm1"] = torch.zeros_like(w["l0.norm1"])
        w["l0.mix.k"][:, 16:] = 0
        w["l0.mix.v"][:, :16] = 0
        w["l0.mix.q"] = w["l0.mix.k"] * 4.0
        w["l0.mix.a2.b"] = torch.full_like(w["l0.mix.a2.b"], 9.0)
        w["l0.mix.a2"] *= 0.1
        w["embed"][2:, :16] *= 0.05
        w["embed"][1, :16] = w["embed"][0, :16]
        w["embed"][1, 16:] = -0.5 * w["embed"][0, 16:]
        w["l0.ls1"] = torch.full_like(w["l0.ls1"], 20.0)      # the mixer's result outweighs the token's own row

    cfg, w = write_model(d, cfg=cfg, ranks={0: 4}, seed=8, edit=edit)
    rng = np.random.RandomState(0)
    for far_at in (0, 7, 8, 200):
        toks = rng.randint(2, 64, size=400).tolist()
        toks[far_at], toks[-1] = 0, 1
        ref = plain.forward(cfg, w, toks).numpy()
        without = plain.forward(cfg, w, toks[:far_at] + [2] + toks[far_at + 1:]).numpy()
        assert np.abs(ref[-1] - without[-1]).max() > 0.15 * np.abs(ref[-1]).max()
        for dtype in ("float32", "bfloat16"):
            eng = engine_of(d, dtype, 8, 448)
            reqs = {"a": toks}
            for steps in (helpers.trace_whole(reqs), helpers.trace_prefill_then_decode(reqs, tail=3),
                          helpers.trace_portions(reqs, sizes=(150, 2, 100, 147, 1))):
                rows = helpers.replay(eng, steps)
                helpers.compare(rows, {"a": ref}, TOL32 if dtype == "float32" else TOL16, f"far token at {far_at}")


@gpu
def test_long_decoding(models):
    """260 tokens one by one: the windows pass over decoded tokens many times, their pages are given back."""
    rng = np.random.RandomState(9)
    for dtype in ("float32", "bfloat16"):
        d, cfg, w, reqs, ref, page = models["A", dtype]
        toks = rng.randint(0, cfg["vocab"], size=260).tolist()
        want = plain.forward(cfg, w, toks).numpy()
        eng = engine_of(d, dtype, page, 320, use_graphs=(dtype == "bfloat16"))
        rows = helpers.replay(eng, helpers.trace_prefill_then_decode({"a": toks}, tail=10 ** 6))
        worst = compare(rows, {"a": want}, dtype, f"long decoding {dtype}")
        print(f"[worst] long decoding, {dtype}: {worst:.3e}")
        assert all(p.used_pages <= 320 // page for p in eng.cache.pools)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(models, dtype):
    """Prompts of unequal length in portions of 7 through ``LLM.generate`` and its scheduler."""
    from ccinfer_b200 import LLM, SamplingParams
    d, cfg, w, reqs, ref, page = models["B", dtype]
    rng = np.random.RandomState(4)
    prompts = [rng.randint(0, cfg["vocab"], size=n).tolist() for n in (1, 9, 20, 33)]
    llm = LLM(d, dtype=dtype, page_size=page, kv_tokens=512, prefill_chunk_size=7, max_requests=4,
              max_tokens_per_step=64)
    got = llm.generate(prompts, SamplingParams(max_tokens=10))
    if dtype == "float32":
        assert got == [plain.greedy(cfg, w, p, 10) for p in prompts]
    else:   # rounding may flip an argmax between two close logits: every token must be (nearly) the best one
        for p, new in zip(prompts, got):
            toks = list(p)
            for t in new:
                row = plain.forward(cfg, w, toks)[-1]
                assert row[t] >= row.max() - 0.05 * row.abs().max()
                toks.append(t)
    assert all(pool.used_pages == 0 for pool in llm.engine.cache.pools)


@gpu
def test_the_programs_as_a_user_calls_them(models, tmp_path):
    """bin/ccinfer: greedy tokens of a model folder; a random model written from a configuration generates the
    same tokens as the same configuration drawn on the device; bin/trace_run: a mixed trace over four request
    slots, its files against the plain logits."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d, cfg, w, reqs, ref, page = models["A", "float32"]
    exe = [sys.executable, os.path.join(root, "bin", "ccinfer")]
    prompt = list(reqs.values())[5]
    r = subprocess.run(exe + ["--model-path", d, "--dtype", "float32", "--page-size", str(page), "--kv-tokens", "256",
                              "--max-tokens", "6", "--prompt-ids", ",".join(map(str, prompt))],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[0])["token_ids"] == plain.greedy(cfg, w, prompt, 6)

    from ccinfer_b200.config.dufizen import DufizenConfig
    full = DufizenConfig.from_json(cfg).with_shapes(plain.tensor_shapes(cfg, plain.CONFIGS["A"][1])).to_json()
    cj = str(tmp_path / "config.json")
    with open(cj, "w") as f:
        json.dump(full, f)
    common = ["--dtype", "float32", "--kv-tokens", "256", "--max-tokens", "5", "--random-prompts", "9,4",
              "--weights-seed", "5", "--weights-std", "0.3"]
    a = subprocess.run(exe + ["--random-config", cj] + common, capture_output=True, text=True, timeout=600)
    assert a.returncode == 0, a.stderr[-2000:]
    made = str(tmp_path / "made")
    wr = subprocess.run(exe + ["--model-path", made, "--write-random-model", cj, "--weights-seed", "5",
                               "--weights-std", "0.3"], capture_output=True, text=True, timeout=600)
    assert wr.returncode == 0, wr.stderr[-2000:]
    b = subprocess.run(exe + ["--model-path", made] + common, capture_output=True, text=True, timeout=600)
    assert b.returncode == 0, b.stderr[-2000:]
    assert a.stdout == b.stdout and len(a.stdout.strip().splitlines()) == 2

    steps = helpers.trace_mixed(reqs, max_live=4, seed=3)
    pool = helpers.max_live_tokens(steps)
    out_dir = tmp_path / "out"
    lines = "".join(json.dumps({"step": i, **st}) + "\n" for i, st in enumerate(steps))
    t = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out",
                        str(out_dir), "--max-tokens", str(pool)], input=lines, capture_output=True, text=True,
                       timeout=600)
    assert t.returncode == 0, t.stderr[-2000:]
    assert t.stdout.split() == [x for i in range(len(steps)) for x in ("done", str(i))]
    rows, seen = {}, {rid: 0 for rid in reqs}
    for i, st in enumerate(steps):
        n_want = sum(len(e["want"]) for e in st["entries"])
        arr = np.fromfile(out_dir / f"{i}.f32", dtype="<f4").reshape(n_want, cfg["vocab"])
        at = 0
        for e in st["entries"]:
            for wnt in e["want"]:
                rows[(e["id"], seen[e["id"]] + wnt)] = arr[at]
                at += 1
            seen[e["id"]] += len(e["tokens"])
    assert len(rows) == sum(len(x) for x in reqs.values())
    helpers.compare(rows, ref, TOL32, "trace_run")


@gpu
def test_a_preempted_request_starts_its_state_again(models):
    """So few pages that a request is preempted and computed again (its slot is closed and opened: the recurrent
    state starts from zero, the windows' pages are taken anew): the greedy tokens are those of a calm run."""
    from ccinfer_b200 import LLM, SamplingParams
    d, cfg, w, reqs, ref, page = models["A", "float32"]
    rng = np.random.RandomState(6)
    prompts = [rng.randint(0, cfg["vocab"], size=n).tolist() for n in (20, 26, 17)]
    llm = LLM(d, dtype="float32", page_size=page, kv_tokens=8 * page, prefill_chunk_size=16, max_requests=4,
              max_tokens_per_step=64)
    got = llm.generate(prompts, [SamplingParams(max_tokens=n) for n in (24, 20, 28)])
    assert llm.scheduler.preemptions > 0
    assert got == [plain.greedy(cfg, w, p, n) for p, n in zip(prompts, (24, 20, 28))]
    llm.engine.cache.check_consistency()
