"""Typed configuration of Dufizen, a decoder whose config.json lists its layers one by one.

    {"architecture": "Dufizen", "vocab": V, "width": D, "norm": {"eps": e},
     "layers": [{"type": T, "mixer": {...}, "mlp": {...} | null}, ...],
     "loop": {"start": a, "stop": b, "times": n},       (optional: layers a .. b-1 run n times in a row)
     "token_side": {"dim": s}}                          (optional: a per-layer token input of s columns)

Mixer types and their keys:

* ``latent_attention``: heads, dim (unrotated query/key coordinates per head), rot_dim (rotated ones), vdim,
  kv_rank, scale, ``rot`` {dims, base}, ``mask`` {size}.
* ``gla``: heads, dim, vdim, tau.  The rank of its narrow decay projection is no key of the file: it is the
  shape of the tensor ``l<i>.mix.a1`` (``with_shapes``); a configuration made in code carries it as ``a_rank``
  and writes it out under that name.

``mlp``: {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "groups": {"count", "keep"}},
"shared": {"ff"}}; ``groups`` and ``shared`` are taken where present.  Nothing here is a default for a size: a
missing key is an error.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Tuple

from ..errors import ModelConfigInvalid
from .tugelorn import _get

ARCHITECTURE = "Dufizen"
LATENT_TYPE = "latent_attention"
GLA_TYPE = "gla"


@dataclasses.dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: int
    rot_dims: int
    rot_base: float
    type: str = LATENT_TYPE


@dataclasses.dataclass(frozen=True)
class GlaMixerConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    a_rank: Optional[int] = None
    type: str = GLA_TYPE


@dataclasses.dataclass(frozen=True)
class MoeConfig:
    experts: int
    top: int
    expert_ff: int
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0
    kind: str = "moe"


@dataclasses.dataclass(frozen=True)
class LayerConfig:
    mixer: object
    mlp: Optional[MoeConfig]

    @property
    def type(self) -> str:
        return self.mixer.type


@dataclasses.dataclass(frozen=True)
class DufizenConfig:
    vocab: int
    width: int
    layers: Tuple[LayerConfig, ...]
    norm_eps: float
    loop: Optional[Tuple[int, int, int]] = None   # (start, stop, times)
    side_dim: Optional[int] = None
    architecture: str = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def run_order(self):
        """[(layer, pass)]: the layers before the loop (pass None), the looped ones ``times`` times, the rest."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        a, b, times = self.loop
        return ([(i, None) for i in range(a)] + [(i, r) for r in range(times) for i in range(a, b)]
                + [(i, None) for i in range(b, n)])

    def with_shapes(self, shapes: dict) -> "DufizenConfig":
        """The sizes that only the tensors give (a checkpoint's name -> shape), filled in."""
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if m.type == GLA_TYPE and m.a_rank is None:
                try:
                    m = dataclasses.replace(m, a_rank=int(shapes[f"l{i}.mix.a1"][0]))
                except (KeyError, IndexError, TypeError):
                    raise ModelConfigInvalid(f"layer {i}: the rank of a1 is neither in config.json nor a tensor "
                                             f"of the checkpoint") from None
                layer = dataclasses.replace(layer, mixer=m)
            layers.append(layer)
        return dataclasses.replace(self, layers=tuple(layers))

    # -- json --------------------------------------------------------------
    @classmethod
    def from_json(cls, j: dict) -> "DufizenConfig":
        vocab, width = _get(j, "vocab", "top", int), _get(j, "width", "top", int)
        eps = _get(j.get("norm"), "eps", "norm", float)
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
            heads, dim, vdim = _get(mj, "heads", mw, int), _get(mj, "dim", mw, int), _get(mj, "vdim", mw, int)
            if t == LATENT_TYPE:
                rot_dim = _get(mj, "rot_dim", mw, int)
                rj = mj.get("rot")
                dims, base = _get(rj, "dims", mw + ".rot", int), _get(rj, "base", mw + ".rot", float)
                if dims % 2 or dims > rot_dim or base <= 0:
                    raise ModelConfigInvalid(f"config.json: {mw}.rot: dims must be even and at most rot_dim, base > 0")
                mixer = LatentMixerConfig(heads, dim, rot_dim, vdim, _get(mj, "kv_rank", mw, int),
                                          _get(mj, "scale", mw, float), _get(mj.get("mask"), "size", mw + ".mask", int),
                                          dims, base)
            elif t == GLA_TYPE:
                tau = _get(mj, "tau", mw, float)
                if tau <= 0:
                    raise ModelConfigInvalid(f"config.json: {mw}.tau must be > 0")
                mixer = GlaMixerConfig(heads, dim, vdim, tau, _get(mj, "a_rank", mw, int) if "a_rank" in mj else None)
            else:
                raise ModelConfigInvalid(f"config.json: {where}.type {t!r} is not one of {(LATENT_TYPE, GLA_TYPE)}")
            mlp = None
            if lj["mlp"] is not None:
                pj = lj["mlp"]
                pw = where + ".mlp"
                if not isinstance(pj, dict) or pj.get("kind") != "moe":
                    raise ModelConfigInvalid(f"config.json: {pw}.kind must be 'moe'")
                rj = pj.get("router")
                experts, top = _get(rj, "experts", pw + ".router", int), _get(rj, "top", pw + ".router", int)
                groups = keep = 1
                if rj.get("groups") is not None:
                    groups = _get(rj["groups"], "count", pw + ".router.groups", int)
                    keep = _get(rj["groups"], "keep", pw + ".router.groups", int)
                if experts % groups or keep > groups or top > (experts // groups) * keep:
                    raise ModelConfigInvalid(f"config.json: {pw}.router: {experts} experts in {groups} groups of which "
                                             f"{keep} are kept cannot give {top}")
                shared = _get(pj["shared"], "ff", pw + ".shared", int) if pj.get("shared") is not None else 0
                mlp = MoeConfig(experts, top, _get(pj.get("expert"), "ff", pw + ".expert", int), groups, keep, shared)
            layers.append(LayerConfig(mixer, mlp))
        loop = None
        if j.get("loop") is not None:
            lp = j["loop"]
            if not isinstance(lp, dict) or isinstance(lp.get("start"), bool) or not isinstance(lp.get("start"), int):
                raise ModelConfigInvalid("config.json: loop.start must be an integer")
            start, stop, times = lp["start"], _get(lp, "stop", "loop", int), _get(lp, "times", "loop", int)
            if not (0 <= start < stop <= len(layers)):
                raise ModelConfigInvalid(f"config.json: loop: 0 <= start < stop <= {len(layers)} is required")
            loop = (start, stop, times)
        side = None
        if j.get("token_side") is not None:
            side = _get(j["token_side"], "dim", "token_side", int)
        return cls(vocab, width, tuple(layers), eps, loop, side)

    def to_json(self) -> dict:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if m.type == LATENT_TYPE:
                mj = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                      "scale": m.scale, "mask": {"size": m.window}, "rot": {"dims": m.rot_dims, "base": m.rot_base}}
            else:
                mj = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "tau": m.tau}
                if m.a_rank is not None:
                    mj["a_rank"] = m.a_rank
            mlp = None
            if layer.mlp is not None:
                p = layer.mlp
                mlp = {"kind": p.kind, "expert": {"ff": p.expert_ff},
                       "router": {"experts": p.experts, "top": p.top, "groups": {"count": p.groups, "keep": p.keep}}}
                if p.shared_ff:
                    mlp["shared"] = {"ff": p.shared_ff}
            layers.append({"type": m.type, "mixer": mj, "mlp": mlp})
        j = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.loop is not None:
            j["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.side_dim is not None:
            j["token_side"] = {"dim": self.side_dim}
        return j
