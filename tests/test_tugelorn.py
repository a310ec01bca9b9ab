"""Tugelorn in the engine against the plain implementation of ``plain_tugelorn``.

Configuration and plan on the CPU; on the GPU each kernel of the design alone, single-layer models of each
mixer, and whole models under every way of cutting the work: whole prompts, token-by-token decoding from the
first token, portions down to two tokens, mixed batches with pages and state slots that are used again,
sharp attention around every window's edge and page border, long decoding, and greedy generation through the
Python entry point and its scheduler.
"""
import copy
import json
import os

import numpy as np
import pytest
import torch

import helpers
import plain_tugelorn as plain

gpu = pytest.mark.gpu

TOL32 = 3e-5          # relative to the largest logit of the request
TOL16 = 6e-2          # (bfloat16 rounding of sharp scores, through up to eight layer runs; seen: 3e-2)
# queries times this: the softmax sits on few keys.  In bfloat16 the rounding of such scores alone moves the
# logits by a tenth of their size, so the weights of the bfloat16 runs are milder
SHARP = {"float32": 4.0, "bfloat16": 1.5}


def write_model(path, name=None, cfg=None, ranks=None, seed=0, sharp=1.0, edit=None):
    from safetensors.torch import save_file
    if cfg is None:
        cfg, ranks, _ = plain.config(name)
    w = plain.random_weights(cfg, ranks, seed, sharp)
    if edit is not None:
        edit(w)
    os.makedirs(path, exist_ok=True)
    save_file({k: v.to(torch.bfloat16) for k, v in w.items()}, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    return cfg, w


def engine_of(path, dtype, page, pool, max_requests=4, use_graphs=False, step_tokens=None):
    from ccinfer_b200.engine.engine import Engine, EngineOptions
    return Engine.from_model_dir(path, EngineOptions(
        dtype=dtype, page_size=page, kv_tokens=pool, max_requests=max_requests,
        max_tokens_per_step=step_tokens or pool, max_context=pool, use_graphs=use_graphs))


def requests_of(cfg, lengths, seed):
    rng = np.random.RandomState(seed)
    return {f"r{i}": rng.randint(0, cfg["vocab"], size=n).tolist() for i, n in enumerate(lengths)}


# ---------------------------------------------------------------------------------------------
# CPU: configuration, plan
# ---------------------------------------------------------------------------------------------
def test_config_is_read_written_and_refused():
    from ccinfer_b200.config.registry import architecture_of
    from ccinfer_b200.config.tugelorn import TugelornConfig
    from ccinfer_b200.errors import ModelConfigInvalid
    cfg, ranks, _ = plain.config("Q")
    assert architecture_of(cfg).name == "Tugelorn"
    c = TugelornConfig.from_json(cfg)
    assert c.loop == (1, 3, 3) and c.residual_mult == 1.0 and c.layers[0].mixer.a_rank is None
    assert c.layers[2].mixer.window == 70 and c.layers[2].mixer.rot.factor is None and not c.layers[2].mixer.bias
    assert c.layers[1].mixer.q_temp == (0.25, 50) and c.layers[1].mixer.bias and c.layers[2].mlp is None
    assert [i for i, _ in c.run_order()] == [0, 1, 2, 1, 2, 1, 2, 3]
    shapes = plain.tensor_shapes(cfg, ranks)
    full = c.with_shapes(shapes)
    assert (full.layers[0].mixer.a_rank, full.layers[0].mixer.g_rank) == (6, 10)
    assert TugelornConfig.from_json(full.to_json()) == full
    with pytest.raises(ModelConfigInvalid):
        c.with_shapes({})
    for damage in (lambda j: j.pop("width"), lambda j: j["norm"].pop("eps"), lambda j: j["layers"][1]["mixer"].pop("scale"),
                   lambda j: j["layers"][0].update(type="attention_3"), lambda j: j["loop"].update(stop=9),
                   lambda j: j["layers"][1]["mixer"].update(heads=3), lambda j: j["layers"][1]["mlp"].update(kind="moe"),
                   lambda j: j["layers"][0]["mixer"].pop("conv")):
        j = copy.deepcopy(cfg)
        damage(j)
        with pytest.raises(ModelConfigInvalid):
            TugelornConfig.from_json(j)


def test_plan_names_every_tensor_and_repeats_the_looped_layers():
    from ccinfer_b200.architectures.tugelorn import build_plan
    from ccinfer_b200.config.tugelorn import TugelornConfig
    for name in plain.CONFIGS:
        cfg, ranks, _ = plain.config(name)
        shapes = plain.tensor_shapes(cfg, ranks)
        plan = build_plan(TugelornConfig.from_json(cfg).with_shapes(shapes))
        plan.validate()
        assert {s.name: tuple(s.shape) for s in plan.tensor_specs()} == shapes
        want = plain.run_order(cfg)
        assert [(e.layer, e.add_embedding) for e in plan.order] == want


def test_heads_are_laid_out_in_a_size_the_kernels_take():
    from ccinfer_b200.parts import GroupedQueryAttention
    assert GroupedQueryAttention.kernel_head_dim(32, 48) == 48
    assert GroupedQueryAttention.kernel_head_dim(64, 128) == 128
    assert GroupedQueryAttention.kernel_head_dim(24, 20) == 32


# ---------------------------------------------------------------------------------------------
# GPU: the kernels alone
# ---------------------------------------------------------------------------------------------
@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [48, 328, 1000])
def test_postnorm_residual_kernel(dtype, D):
    from ccinfer_b200 import kernels
    g = torch.Generator().manual_seed(D)
    T = 7
    h, add = torch.randn(T, D, generator=g), torch.randn(T, D, generator=g)
    delta = (3 * torch.randn(T, D, generator=g)).to(dtype)
    w1, w2 = 1 + 0.3 * torch.randn(D, generator=g), 1 + 0.3 * torch.randn(D, generator=g)
    want_h = h.double() + 0.4 * plain.rms_norm(delta.double(), w1.double(), 1e-5) + add.double()
    want_y = plain.rms_norm(want_h, w2.double(), 1e-5)
    hd, y = h.cuda(), torch.empty(T, D, dtype=dtype, device="cuda")
    kernels.postnorm_residual(hd, delta.cuda(), w1.cuda(), 0.4, 1e-5, add=add.cuda(), y=y, w_next=w2.cuda(), eps_next=1e-5)
    assert (hd.cpu().double() - want_h).abs().max() < 2e-6 * want_h.abs().max()
    tol = 1e-6 if dtype == torch.float32 else 8e-3
    assert (y.cpu().double() - want_y).abs().max() < tol * want_y.abs().max()
    # the sum alone, and the addition alone
    h2 = h.cuda()
    kernels.postnorm_residual(h2, delta.cuda(), w1.cuda(), 1.0, 1e-5)
    assert (h2.cpu().double() - (h.double() + plain.rms_norm(delta.double(), w1.double(), 1e-5))).abs().max() < 1e-5
    h3 = h.cuda()
    kernels.postnorm_residual(h3, None, None, 0.0, 0.0, add=add.cuda())
    assert torch.equal(h3.cpu(), h + add)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("F,block", [(64, 64), (128, 64), (50, 0)])
def test_clamped_glu_kernel(dtype, F, block):
    from ccinfer_b200 import kernels
    g = torch.Generator().manual_seed(F)
    gate, up = (3 * torch.randn(5, F, generator=g)).to(dtype), (3 * torch.randn(5, F, generator=g)).to(dtype)
    if block:
        gu = torch.cat([gate.view(5, F // block, block), up.view(5, F // block, block)], dim=2).reshape(5, 2 * F)
    else:
        gu = torch.cat([gate, up], dim=1)
    act = torch.empty(5, F, dtype=dtype, device="cuda")
    kernels.clamped_glu(act, gu.contiguous().cuda(), block, 2.5, 1.702, 1.0)
    want = plain.clamped_glu(gate.double(), up.double(), 2.5)
    assert (act.cpu().double() - want).abs().max() < (1e-6 if dtype == torch.float32 else 1e-2) * want.abs().max()


@gpu
@pytest.mark.parametrize("kind,M,F,K", [("tc", 1, 9600, 256), ("tc", 16, 9600, 64), ("fewrows", 3, 256, 512),
                                        ("fewrows", 16, 128, 2048), ("pair", 300, 256, 256), ("pair", 1100, 192, 512)])
def test_clamped_glu_as_the_epilogue_of_the_product(kind, M, F, K):
    from ccinfer_b200 import kernels
    g = torch.Generator().manual_seed(M + F)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    wg = (torch.randn(F, K, generator=g) * 2.0 / K ** 0.5).to(torch.bfloat16)
    wu = (torch.randn(F, K, generator=g) * 2.0 / K ** 0.5).to(torch.bfloat16)
    w = kernels.interleave_gate_up(wg.cuda(), wu.cuda(), kernels.SWIGLU_BLOCK)
    act = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
    kernels.gemm_glu_bf16(act, x.cuda(), w, 1.5, 1.702, 1.0, kind)
    want = plain.clamped_glu(x.double() @ wg.double().T, x.double() @ wu.double().T, 1.5)
    assert (act.cpu().double() - want).abs().max() < 2e-2 * max(1.0, want.abs().max())


@gpu
@pytest.mark.parametrize("H,G,dk,dv", [(2, 1, 8, 8), (3, 3, 24, 40), (4, 2, 64, 70), (2, 2, 130, 33), (1, 1, 256, 16)])
def test_delta_recurrence_kernel_carries_its_state(H, G, dk, dv):
    """Two requests in unequal portions over three launches, slots 2 and 0 of a state of three."""
    from ccinfer_b200 import kernels
    g = torch.Generator().manual_seed(dk)
    lens = [37, 20]
    seqs = []
    for n in lens:
        q = plain.unit_rows(torch.randn(n, G, dk, generator=g, dtype=torch.float64)) * dk ** -0.5
        k = plain.unit_rows(torch.randn(n, G, dk, generator=g, dtype=torch.float64))
        v = torch.randn(n, H, dv, generator=g, dtype=torch.float64)
        beta = torch.rand(n, H, generator=g, dtype=torch.float64)
        decay = 0.5 + 0.5 * torch.rand(n, H, dk, generator=g, dtype=torch.float64)
        rep = H // G
        want = plain.delta_rule(q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1), v, beta, decay)
        seqs.append((q, k, v, beta, decay, want))
    state = torch.full((3, H, dv, dk), 7.0, device="cuda")
    state[2].zero_()
    state[0].zero_()
    slots = torch.tensor([2, 0], dtype=torch.int32, device="cuda")
    cursor = [0, 0]
    for portion in ([17, 1], [1, 16], [19, 3]):
        rows = [[t[cursor[i]:cursor[i] + n].float() for t in seqs[i][:5]] for i, n in enumerate(portion)]
        cat = [torch.cat([r[j] for r in rows]).contiguous().cuda() for j in range(5)]
        cu = torch.tensor([0, portion[0], sum(portion)], dtype=torch.int32, device="cuda")
        out = torch.empty(sum(portion), H, dv, device="cuda")
        kernels.delta_recurrence(cat[0], cat[1], cat[2], cat[4], cat[3], state, out, cu, slots, 2, G, H, dk, dv)
        got = out.cpu().double()
        at = 0
        for i, n in enumerate(portion):
            want = seqs[i][5][cursor[i]:cursor[i] + n]
            assert (got[at:at + n] - want).abs().max() < 2e-5 * max(1.0, want.abs().max())
            at += n
            cursor[i] += n
    assert torch.all(state[1] == 7.0)   # a slot of no request in the step is left alone


# ---------------------------------------------------------------------------------------------
# GPU: one layer of each kind
# ---------------------------------------------------------------------------------------------
SINGLE = {
    "window, rotation": (plain._attn(4, 2, 16, 32, 0.3, window=9, rot=(8, 1000.0, 4.0)), None),
    "rotation of the whole head": (plain._attn(2, 2, 32, 32, 0.2, rot=(32, 10000.0, None)), None),
    "biases, temperature": (plain._attn(6, 3, 32, 16, 0.2, q_temp=(0.7, 5), kind="attention_2"), None),
    "delta": (plain._delta(4, 2, 24, 20, 4), None),
    "delta, feed-forward": (plain._delta(2, 2, 8, 16, 2), plain._mlp(72, 1.0)),
}


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", list(SINGLE))
def test_one_layer_of_each_kind(tmp_path, kind, dtype):
    cfg = plain._model(40, 97, 1e-5, 0.7, [SINGLE[kind]])
    ranks = {0: (5, 12)}
    d = str(tmp_path / "m")
    cfg, w = write_model(d, cfg=cfg, ranks=ranks, seed=3, sharp=3.0 if dtype == "float32" else 1.5)
    reqs = requests_of(cfg, [1, 2, 31, 50], 1)
    ref = {rid: plain.forward(cfg, w, t).numpy() for rid, t in reqs.items()}
    eng = engine_of(d, dtype, 8, 256)
    for steps in (helpers.trace_whole(reqs), helpers.trace_prefill_then_decode(reqs, tail=64),
                  helpers.trace_portions(reqs, sizes=(2, 5, 3, 2, 11))):
        rows = helpers.replay(eng, steps)
        worst = helpers.compare(rows, ref, TOL32 if dtype == "float32" else TOL16, f"{kind} {dtype}")
        print(f"[worst] one layer, {kind}, {dtype}: {worst:.3e}")


# ---------------------------------------------------------------------------------------------
# GPU: whole models under every cutting
# ---------------------------------------------------------------------------------------------
LENGTHS = {"P": [1, 2, 23, 24, 25, 26, 60, 97], "Q": [3, 69, 70, 71, 72, 140, 200], "R": [1, 15, 16, 17, 18, 33, 64],
           "S": [1, 4, 5, 6, 7, 21, 50]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name in plain.CONFIGS:
        for dtype, sharp in SHARP.items():
            d = str(tmp_path_factory.mktemp("tug" + name))
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
    """Prompt lengths sit just below, at and just above every window and page border of the configuration, and
    the attention is sharp (queries times four in the 32-bit runs), so a key one place off shows."""
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
    worst = helpers.compare(rows, ref, TOL32 if dtype == "float32" else TOL16, f"{name} {dtype} {mode}")
    print(f"[worst] {name}, {dtype}, {mode}: {worst:.3e}")
    eng.cache.check_consistency()
    assert all(p.used_pages == 0 for p in eng.cache.pools)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_and_graphs(models, dtype):
    """Portions of more than 64 tokens after a cached prefix beside decode steps replayed from CUDA graphs."""
    d, cfg, w, reqs, ref, page = models["Q", dtype]
    steps = helpers.trace_mixed(reqs, max_live=3, seed=13, prefill_frac=0.8, portion_choices=(70, 130, 65, 2, 100))
    pool = helpers.max_live_tokens(steps, round_to=64)
    eng = engine_of(d, dtype, page, pool, max_requests=4, use_graphs=True)
    rows = helpers.replay(eng, steps)
    worst = helpers.compare(rows, ref, TOL32 if dtype == "float32" else TOL16, f"Q {dtype} long portions, graphs")
    print(f"[worst] Q, {dtype}, long portions, graphs: {worst:.3e}")
    assert eng.graph_replays > 0


@gpu
def test_a_slot_that_is_used_again_starts_from_zero(models):
    """Two state slots, five requests one after another and in pairs: every later request gets a slot whose
    state an earlier one left behind."""
    d, cfg, w, reqs, ref, page = models["P", "float32"]
    eng = engine_of(d, "float32", page, 256, max_requests=2)
    ids = list(reqs)[3:8]
    order = [[ids[0]], [ids[1], ids[2]], [ids[3], ids[4]]]
    for group in order:
        steps = helpers.trace_mixed({r: reqs[r] for r in group}, max_live=2, seed=1)
        rows = helpers.replay(eng, steps)
        helpers.compare(rows, ref, TOL32, "slots used again")
    assert eng.cache.slots.free_slots == 2


@gpu
def test_a_far_key_decides(tmp_path):
    """One layer that sees everything.  Queries and keys read the first half of the stream (the query projection
    is twice the key projection), values the second half, and tokens 0 and 1 have the same first half: the query
    of token 1 then matches the key of token 0 as well as its own and hardly any other.  Token 0 stands at ONE
    far place among 300 and token 1 at the end: the last position's logits follow the far token's value, and
    dropping or misplacing its key would change them by their own size.  The far place is the first token, the
    last of a page, the first of the next, and the middle."""
    cfg = plain._model(32, 64, 1e-5, 1.0, [(plain._attn(2, 1, 16, 16, 1.0, q_temp=(0.2, 48), kind="attention_2"), None)])
    d = str(tmp_path / "far")

    def edit(w):
        w["l0.norm1"] = torch.ones_like(w["l0.norm1"])
        w["l0.mix.k"][:, 16:] = 0
        w["l0.mix.v"][:, :16] = 0
        w["l0.mix.q"] = torch.cat([w["l0.mix.k"], w["l0.mix.k"]]) * 2.0
        w["l0.mix.q.b"] = torch.zeros_like(w["l0.mix.q.b"])
        w["l0.mix.k.b"] = torch.zeros_like(w["l0.mix.k.b"])
        w["embed"][1, :16] = w["embed"][0, :16]

    cfg, w = write_model(d, cfg=cfg, ranks={}, seed=8, edit=edit)
    rng = np.random.RandomState(0)
    for far_at in (0, 7, 8, 150):
        toks = rng.randint(2, 64, size=300).tolist()
        toks[far_at], toks[-1] = 0, 1
        ref = plain.forward(cfg, w, toks).numpy()
        without = plain.forward(cfg, w, toks[:far_at] + [2] + toks[far_at + 1:]).numpy()
        assert np.abs(ref[-1] - without[-1]).max() > 0.2 * np.abs(ref[-1]).max()   # the far key does decide
        for dtype in ("float32", "bfloat16"):
            eng = engine_of(d, dtype, 8, 320)
            reqs = {"a": toks}
            for steps in (helpers.trace_whole(reqs), helpers.trace_prefill_then_decode(reqs, tail=3),
                          helpers.trace_portions(reqs, sizes=(150, 2, 100, 47, 1))):
                rows = helpers.replay(eng, steps)
                helpers.compare(rows, {"a": ref}, TOL32 if dtype == "float32" else TOL16, f"far key at {far_at}")


@gpu
def test_long_decoding(models):
    """260 tokens one by one: the window of 24 passes over decoded tokens many times, its pages are given back."""
    rng = np.random.RandomState(9)
    for dtype in ("float32", "bfloat16"):
        d, cfg, w, reqs, ref, page = models["P", dtype]
        toks = rng.randint(0, cfg["vocab"], size=260).tolist()
        want = plain.forward(cfg, w, toks).numpy()
        eng = engine_of(d, dtype, page, 320, use_graphs=(dtype == "bfloat16"))
        rows = helpers.replay(eng, helpers.trace_prefill_then_decode({"a": toks}, tail=10 ** 6))
        worst = helpers.compare(rows, {"a": want}, TOL32 if dtype == "float32" else TOL16, f"long decoding {dtype}")
        print(f"[worst] long decoding, {dtype}: {worst:.3e}")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(models, dtype):
    """Prompts of unequal length in portions of 7 through ``LLM.generate`` and its scheduler."""
    from ccinfer_b200 import LLM, SamplingParams
    d, cfg, w, reqs, ref, page = models["R", dtype]
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
    """bin/ccinfer: greedy tokens of a model folder, and a random model written from a configuration (which
    must carry the delta rule's ranks) that generates the same tokens as the same configuration drawn on the
    device; bin/trace_run: a mixed trace over four request slots, its files against the plain logits."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d, cfg, w, reqs, ref, page = models["R", "float32"]
    exe = [sys.executable, os.path.join(root, "bin", "ccinfer")]
    prompt = list(reqs.values())[2]
    r = subprocess.run(exe + ["--model-path", d, "--dtype", "float32", "--page-size", str(page), "--kv-tokens", "256",
                              "--max-tokens", "6", "--prompt-ids", ",".join(map(str, prompt))],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[0])["token_ids"] == plain.greedy(cfg, w, prompt, 6)

    from ccinfer_b200.config.tugelorn import TugelornConfig
    full = TugelornConfig.from_json(cfg).with_shapes(plain.tensor_shapes(cfg, plain.CONFIGS["R"][1])).to_json()
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
    with open(cj, "w") as f:
        json.dump(cfg, f)   # without the ranks no random model can be drawn: the error says so
    bad = subprocess.run(exe + ["--random-config", cj] + common, capture_output=True, text=True, timeout=600)
    assert bad.returncode == 2 and "ranks" in bad.stderr

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
    """So few pages that a request is preempted and computed again (its slot is closed and opened: the delta
    rule's state and the convolution's rows start from zero): the greedy tokens are those of a calm run."""
    from ccinfer_b200 import LLM, SamplingParams
    d, cfg, w, reqs, ref, page = models["R", "float32"]
    rng = np.random.RandomState(6)
    prompts = [rng.randint(0, cfg["vocab"], size=n).tolist() for n in (20, 26, 17)]
    llm = LLM(d, dtype="float32", page_size=page, kv_tokens=6 * page, prefill_chunk_size=16, max_requests=4,
              max_tokens_per_step=64)
    got = llm.generate(prompts, [SamplingParams(max_tokens=n) for n in (24, 20, 28)])
    assert llm.scheduler.preemptions > 0
    assert got == [plain.greedy(cfg, w, p, n) for p, n in zip(prompts, (24, 20, 28))]
    llm.engine.cache.check_consistency()
