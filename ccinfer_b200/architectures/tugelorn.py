"""Tugelorn put together from the parts: every layer of its own kind, some of them run several times.

A layer is a ``SandwichNormBlock`` (a norm before and after each sublayer, the normed output times
``residual_mult``) around one of three mixers (softmax attention over a window with rotated interleaved
pairs; softmax attention over everything with biases and a query temperature; the gated delta rule with a
decay per key channel) and, where the layer has one, a gated feed-forward with clamped inputs.  A loop over
some layers becomes repeated entries of the running order: each run has a cache or state of its own, and the
first layer of every pass but the first adds the embedding's rows to the stream again.

Tensor names: ``embed``, ``l<i>.norm1 / norm1b / norm2 / norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.gate / up / down``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.tugelorn import DELTA_TYPE, TugelornConfig
from ..engine.plan import ModelPlan, RunEntry
from ..errors import ModelConfigInvalid
from ..parts import (ChannelGatedDelta, ClampedGLU, GroupedQueryAttention, OutputHead, QueryTemperature, RMSNorm,
                     RotaryHalf, SandwichNormBlock, TokenEmbedding)
from ..parts.position import NoPosition

GLU_SLOPE = 1.702    # the feed-forward's gate is g * sigmoid(1.702 g) ...
GLU_UP_SHIFT = 1.0   # ... times (u + 1)

# The tensor-core attention kernels round the softmax weights to bfloat16 for their product with the values;
# True sends every row to the kernel that keeps them float.
FLOAT_ATTENTION_WEIGHTS = False


def _attention(cfg: TugelornConfig, m, p: str):
    hd = GroupedQueryAttention.kernel_head_dim(m.dim, m.vdim)
    q_temp = QueryTemperature(*m.q_temp) if m.q_temp is not None else None
    if m.rot is not None:
        position = RotaryHalf(hd, m.rot.base, rotary_dim=m.rot.dims, interleaved=True,
                              linear_scaling=m.rot.factor if m.rot.factor is not None else 1.0,
                              query_temperature=None if q_temp is None else q_temp.query_temperature())
    else:
        position = q_temp if q_temp is not None else NoPosition()
    names = {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"}
    if m.bias:
        names.update(q_bias=p + "q.b", k_bias=p + "k.b", v_bias=p + "v.b")
    return GroupedQueryAttention(hidden=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
                                 position=position, names=names, window=m.window, scale=m.scale, value_dim=m.vdim,
                                 float_weights=FLOAT_ATTENTION_WEIGHTS)


def _delta(cfg: TugelornConfig, m, p: str, layer: int):
    if m.a_rank is None or m.g_rank is None:
        raise ModelConfigInvalid(f"layer {layer}: the ranks of the narrow projections are unknown "
                                 f"(TugelornConfig.with_shapes fills them in from a checkpoint)")
    names = {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o", "q_conv": p + "q.conv", "k_conv": p + "k.conv",
             "v_conv": p + "v.conv", "b": p + "b", "A_log": p + "A_log", "dt_bias": p + "dt_bias", "a1": p + "a1",
             "a2": p + "a2", "g1": p + "g1", "g2": p + "g2", "norm": p + "norm", "a_rank": m.a_rank,
             "g_rank": m.g_rank}
    return ChannelGatedDelta(cfg.width, m.heads, m.kv_heads, m.dim, m.vdim, m.conv, cfg.norm_eps, names)


def build_plan(cfg: TugelornConfig) -> ModelPlan:
    D, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        mixer = _delta(cfg, m, p + "mix.", i) if m.type == DELTA_TYPE else _attention(cfg, m, p + "mix.")
        norm2 = ffn = post2 = None
        if layer.mlp is not None:
            norm2, post2 = RMSNorm(D, eps, p + "norm2"), RMSNorm(D, eps, p + "norm2b")
            ffn = ClampedGLU(D, layer.mlp.ff, {"gate": p + "mlp.gate", "up": p + "mlp.up", "down": p + "mlp.down"},
                             limit=layer.mlp.limit, alpha=GLU_SLOPE, shift=GLU_UP_SHIFT)
        layers.append(SandwichNormBlock(RMSNorm(D, eps, p + "norm1"), mixer, RMSNorm(D, eps, p + "norm1b"),
                                        norm2, ffn, post2, mult=cfg.residual_mult))
    first_of_pass = cfg.loop[0] if cfg.loop is not None else None
    order = [RunEntry(i, add_embedding=(r > 0 and i == first_of_pass)) for i, r in cfg.run_order()]
    return ModelPlan(embedding=TokenEmbedding(cfg.vocab, D, "embed"), layers=layers, order=order,
                     final_norm=RMSNorm(D, eps, "final.norm"), head=OutputHead(D, cfg.vocab, "head"),
                     vocab_size=cfg.vocab, max_position=None)
