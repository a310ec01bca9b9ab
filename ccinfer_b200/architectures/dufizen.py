"""Dufizen put together from the parts: latent attention and gated linear attention layers with mixtures of
experts, a factor per channel on every sublayer's output, a per-layer token input, and a loop over some layers.

A layer is a ``LayerScaleBlock``: h += ls1 * mixer(norm1(h)); h += ls2 * moe(norm2(h)); h += side(h, token), the
norms RMS norms whose stored weights lie around zero (the factor is 1 + w).  A loop over some layers becomes
repeated entries of the running order, each run with a cache or state of its own; every pass (the first too)
enters through ``LoopInput``: h <- Win [h | embedding rows] + step[pass].  The head is the embedding table.

Tensor names: ``embed``, ``side.embed``, ``loop.in``, ``loop.step``, ``l<i>.norm1 / norm2 / ls1 / ls2``,
``l<i>.mix.*``, ``l<i>.mlp.router / correction / e<k>.up / e<k>.down / shared.up / shared.down``,
``l<i>.side.gate / proj / norm``, ``final.norm``.
"""
from __future__ import annotations

from ..config.dufizen import GLA_TYPE, DufizenConfig
from ..engine.plan import ModelPlan, RunEntry
from ..errors import ModelConfigInvalid
from ..parts import (GatedLinearAttention, LatentAttention, LayerScaleBlock, LoopInput, MixtureOfExperts, OutputHead,
                     RMSNorm, TokenEmbedding, TokenSideInput)

NORM_WEIGHT_OFFSET = 1.0   # the model's norms multiply by (1 + w)


def _mixer(cfg: DufizenConfig, m, p: str, layer: int):
    if m.type == GLA_TYPE:
        if m.a_rank is None:
            raise ModelConfigInvalid(f"layer {layer}: the rank of the narrow decay projection is unknown "
                                     f"(DufizenConfig.with_shapes fills it in from a checkpoint)")
        names = {"q": p + "q", "k": p + "k", "v": p + "v", "g": p + "g", "o": p + "o", "norm": p + "norm",
                 "a1": p + "a1", "a2": p + "a2", "a2_bias": p + "a2.b"}
        return GatedLinearAttention(cfg.width, m.heads, m.dim, m.vdim, m.tau, m.a_rank, cfg.norm_eps, names)
    names = {"q": p + "q", "dkv": p + "dkv", "dkv_norm": p + "dkv.norm", "uk": p + "uk", "uv": p + "uv",
             "sink": p + "sink", "g": p + "g", "o": p + "o"}
    return LatentAttention(cfg.width, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.window, m.scale, m.rot_base,
                           m.rot_dims, cfg.norm_eps, names)


def build_plan(cfg: DufizenConfig) -> ModelPlan:
    D, eps = cfg.width, cfg.norm_eps
    n_layers = len(cfg.layers)

    def norm(name):
        return RMSNorm(D, eps, name, weight_offset=NORM_WEIGHT_OFFSET)

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        norm2 = ffn = None
        if layer.mlp is not None:
            q = layer.mlp
            names = {"router": p + "mlp.router", "correction": p + "mlp.correction", "up": p + "mlp.e{e}.up",
                     "down": p + "mlp.e{e}.down", "shared_up": p + "mlp.shared.up", "shared_down": p + "mlp.shared.down"}
            norm2 = norm(p + "norm2")
            ffn = MixtureOfExperts(D, q.experts, q.top, q.expert_ff, names, q.groups, q.keep, q.shared_ff)
        side = None
        if cfg.side_dim is not None:
            side = TokenSideInput(cfg.vocab, D, cfg.side_dim, i * cfg.side_dim, n_layers * cfg.side_dim, eps,
                                  {"table": "side.embed", "gate": p + "side.gate", "proj": p + "side.proj",
                                   "norm": p + "side.norm"})
        layers.append(LayerScaleBlock(D, norm(p + "norm1"), _mixer(cfg, layer.mixer, p + "mix.", i),
                                      (p + "ls1", p + "ls2"), norm2, ffn, side))
    extras = []
    enter = None
    if cfg.loop is not None:
        enter = LoopInput(D, cfg.loop[2], {"in": "loop.in", "step": "loop.step"})
        extras.append(enter)
    order = []
    for i, r in cfg.run_order():
        first = r is not None and i == cfg.loop[0]
        order.append(RunEntry(i, enter=enter if first else None, enter_number=r if first else 0))
    return ModelPlan(embedding=TokenEmbedding(cfg.vocab, D, "embed"), layers=layers, order=order,
                     final_norm=norm("final.norm"), head=OutputHead(D, cfg.vocab, "embed"), vocab_size=cfg.vocab,
                     max_position=None, extras=extras)
