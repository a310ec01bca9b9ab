"""Typed configuration of Tugelorn, a decoder whose config.json lists its layers one by one.

    {"architecture": "Tugelorn", "vocab": V, "width": D, "norm": {"eps": e}, "residual_mult": m,
     "layers": [{"type": T, "mixer": {...}, "mlp": {"kind": "dense", "ff": F, "limit": L} | null}, ...],
     "loop": {"start": a, "stop": b, "times": n}}          (optional: layers a .. b-1 run n times in a row)

Mixer types and their keys:

* ``attention``: heads, kv_heads, dim, vdim, scale; ``rot`` {dims, base, scaling {factor}} (rotation of
  interleaved pairs over the first ``dims`` coordinates, frequencies divided by ``factor``); ``mask`` {size}
  (a query sees itself and the size - 1 tokens before it).  No biases.
* ``attention_2``: heads, kv_heads, dim, vdim, scale; biases on q, k, v; no rotation; ``q_temp`` {coef, every}
  (queries grow with the logarithm of the position); every earlier token is seen.
* ``channel_delta``: heads, kv_heads, dim, vdim, conv (taps): the gated delta rule with a decay per key
  channel (``parts.delta``).  The ranks of its two narrow projection pairs are no keys of the file: they are
  the shapes of the tensors ``l<i>.mix.a1`` and ``l<i>.mix.g1`` (``with_shapes``); a configuration made in
  code carries them as ``a_rank`` and ``g_rank`` and writes them out under these names.

The sub-objects ``rot``, ``rot.scaling``, ``mask`` and ``q_temp`` are taken where they are present on either
attention type; what a type always has is its biases.  Nothing here is a default for a size: a missing key is
an error.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Tuple

from ..errors import ModelConfigInvalid

ARCHITECTURE = "Tugelorn"
ATTENTION_TYPES = ("attention", "attention_2")
DELTA_TYPE = "channel_delta"


def _get(j, key, where, kind):
    if not isinstance(j, dict) or key not in j:
        raise ModelConfigInvalid(f"config.json: {where}: required key '{key}' is missing")
    v = j[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int) or not (0 < v < 2 ** 31):
            raise ModelConfigInvalid(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
        return v
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ModelConfigInvalid(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclasses.dataclass(frozen=True)
class Rotation:
    dims: int
    base: float
    factor: Optional[float] = None   # linear scaling: frequencies divided by it


@dataclasses.dataclass(frozen=True)
class AttentionMixerConfig:
    type: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[Rotation] = None
    window: Optional[int] = None
    q_temp: Optional[Tuple[float, int]] = None   # (coef, every)

    @property
    def bias(self) -> bool:
        return self.type == "attention_2"


@dataclasses.dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    a_rank: Optional[int] = None
    g_rank: Optional[int] = None
    type: str = DELTA_TYPE


@dataclasses.dataclass(frozen=True)
class MlpConfig:
    ff: int
    limit: float
    kind: str = "dense"


@dataclasses.dataclass(frozen=True)
class LayerConfig:
    mixer: object
    mlp: Optional[MlpConfig]

    @property
    def type(self) -> str:
        return self.mixer.type


@dataclasses.dataclass(frozen=True)
class TugelornConfig:
    vocab: int
    width: int
    layers: Tuple[LayerConfig, ...]
    norm_eps: float
    residual_mult: float
    loop: Optional[Tuple[int, int, int]] = None   # (start, stop, times)
    architecture: str = ARCHITECTURE

    # -- derived -----------------------------------------------------------
    @property
    def vocab_size(self) -> int:
        return self.vocab

    def run_order(self):
        """[(layer, pass)]: the layers before the loop, the looped ones ``times`` times, the rest."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, 0) for i in range(n)]
        a, b, times = self.loop
        return ([(i, 0) for i in range(a)] + [(i, r) for r in range(times) for i in range(a, b)]
                + [(i, 0) for i in range(b, n)])

    def with_shapes(self, shapes: dict) -> "TugelornConfig":
        """The sizes that only the tensors give (a checkpoint's name -> shape), filled in."""
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if m.type == DELTA_TYPE and (m.a_rank is None or m.g_rank is None):
                try:
                    a, g = shapes[f"l{i}.mix.a1"], shapes[f"l{i}.mix.g1"]
                    m = dataclasses.replace(m, a_rank=int(a[0]), g_rank=int(g[0]))
                except (KeyError, IndexError, TypeError):
                    raise ModelConfigInvalid(f"layer {i}: the ranks of a1 and g1 are neither in config.json nor "
                                             f"tensors of the checkpoint") from None
                layer = dataclasses.replace(layer, mixer=m)
            layers.append(layer)
        return dataclasses.replace(self, layers=tuple(layers))

    # -- json --------------------------------------------------------------
    @classmethod
    def from_json(cls, j: dict) -> "TugelornConfig":
        vocab, width = _get(j, "vocab", "top", int), _get(j, "width", "top", int)
        eps = _get(j.get("norm"), "eps", "norm", float)
        mult = _get(j, "residual_mult", "top", float)
        if eps <= 0:
            raise ModelConfigInvalid("config.json: norm.eps must be > 0")
        raw = j.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ModelConfigInvalid("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, lj in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(lj, dict) or "type" not in lj or "mixer" not in lj or "mlp" not in lj:
                raise ModelConfigInvalid(f"config.json: {where} needs 'type', 'mixer' and 'mlp' (null for none)")
            t, mj = lj["type"], lj["mixer"]
            mw = where + ".mixer"
            heads, kv = _get(mj, "heads", mw, int), _get(mj, "kv_heads", mw, int)
            dim, vdim = _get(mj, "dim", mw, int), _get(mj, "vdim", mw, int)
            if heads % kv:
                raise ModelConfigInvalid(f"config.json: {mw}: heads {heads} is not a multiple of kv_heads {kv}")
            if t in ATTENTION_TYPES:
                rot = window = q_temp = None
                if mj.get("rot") is not None:
                    rj = mj["rot"]
                    factor = None
                    if rj.get("scaling") is not None:
                        factor = _get(rj["scaling"], "factor", mw + ".rot.scaling", float)
                        if factor <= 0:
                            raise ModelConfigInvalid(f"config.json: {mw}.rot.scaling.factor must be > 0")
                    rot = Rotation(_get(rj, "dims", mw + ".rot", int), _get(rj, "base", mw + ".rot", float), factor)
                    if rot.dims % 2 or rot.dims > dim or rot.base <= 0:
                        raise ModelConfigInvalid(f"config.json: {mw}.rot: dims must be even and at most dim, base > 0")
                if mj.get("mask") is not None:
                    window = _get(mj["mask"], "size", mw + ".mask", int)
                if mj.get("q_temp") is not None:
                    q_temp = (_get(mj["q_temp"], "coef", mw + ".q_temp", float),
                              _get(mj["q_temp"], "every", mw + ".q_temp", int))
                mixer = AttentionMixerConfig(t, heads, kv, dim, vdim, _get(mj, "scale", mw, float), rot, window, q_temp)
            elif t == DELTA_TYPE:
                ranks = {k: (_get(mj, k, mw, int) if k in mj else None) for k in ("a_rank", "g_rank")}
                mixer = DeltaMixerConfig(heads, kv, dim, vdim, _get(mj, "conv", mw, int), **ranks)
            else:
                raise ModelConfigInvalid(f"config.json: {where}.type {t!r} is not one of "
                                         f"{ATTENTION_TYPES + (DELTA_TYPE,)}")
            mlp = None
            if lj["mlp"] is not None:
                pj = lj["mlp"]
                if not isinstance(pj, dict) or pj.get("kind") != "dense":
                    raise ModelConfigInvalid(f"config.json: {where}.mlp.kind must be 'dense'")
                mlp = MlpConfig(_get(pj, "ff", where + ".mlp", int), _get(pj, "limit", where + ".mlp", float))
                if mlp.limit <= 0:
                    raise ModelConfigInvalid(f"config.json: {where}.mlp.limit must be > 0")
            layers.append(LayerConfig(mixer, mlp))
        loop = None
        if j.get("loop") is not None:
            lp = j["loop"]
            if not isinstance(lp, dict) or isinstance(lp.get("start"), bool) or not isinstance(lp.get("start"), int):
                raise ModelConfigInvalid("config.json: loop.start must be an integer")
            start, stop, times = lp["start"], _get(lp, "stop", "loop", int), _get(lp, "times", "loop", int)
            if not (0 <= start < stop <= len(layers)):
                raise ModelConfigInvalid(f"config.json: loop: 0 <= start < stop <= {len(layers)} is required")
            if start == 0 and times > 1:
                pass   # the first pass starts from the embedding alone; later ones add it again
            loop = (start, stop, times)
        return cls(vocab, width, tuple(layers), eps, mult, loop)

    def to_json(self) -> dict:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            mj = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim}
            if m.type == DELTA_TYPE:
                mj["conv"] = m.conv
                if m.a_rank is not None:
                    mj["a_rank"], mj["g_rank"] = m.a_rank, m.g_rank
            else:
                mj["scale"] = m.scale
                if m.rot is not None:
                    mj["rot"] = {"dims": m.rot.dims, "base": m.rot.base}
                    if m.rot.factor is not None:
                        mj["rot"]["scaling"] = {"factor": m.rot.factor}
                if m.window is not None:
                    mj["mask"] = {"size": m.window}
                if m.q_temp is not None:
                    mj["q_temp"] = {"coef": m.q_temp[0], "every": m.q_temp[1]}
            mlp = None if layer.mlp is None else {"kind": layer.mlp.kind, "ff": layer.mlp.ff, "limit": layer.mlp.limit}
            layers.append({"type": m.type, "mixer": mj, "mlp": mlp})
        j = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "layers": layers}
        if self.loop is not None:
            j["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return j
