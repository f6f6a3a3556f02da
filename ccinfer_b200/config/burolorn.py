"""Typed configuration of Burolorn, a decoder whose config.json lists its layers one by one.

    {"architecture": "Burolorn", "vocab": V, "width": D, "norm": {"eps": e}, "logit_scale": s,
     "layers": [{"type": "attention", "mixer": {...}, "mlp": {...} | null}, ...],
     "token_side": {"dim": n}}                           (optional: a per-layer token input of n columns)

The mixer ``attention``: heads, kv_heads, dim (query/key size of a head), vdim (value size), scale; ``conv`` (taps
of a short causal convolution on q, k and v; absent, null or 0: none); ``rot`` {dims, base} (rotate-half over the
first ``dims`` coordinates; absent: no rotation); ``mask`` {size} (a query sees the keys of its own run of ``size``
positions; absent: every earlier key); ``v_mix`` (true: values are mixed with those of the first such layer).

``mlp``: {"kind": "dense", "ff": F} or {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale",
"groups": {"count", "keep"}}, "shared": {"ff"}}; ``groups``, ``scale`` and ``shared`` are taken where present.
Nothing here is a default for a size: a missing key is an error.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Tuple

from ..errors import ModelConfigInvalid
from .tugelorn import _get

ARCHITECTURE = "Burolorn"
ATTENTION_TYPE = "attention"


@dataclasses.dataclass(frozen=True)
class MixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int = 0                       # taps; 0: no convolution
    rot_dims: int = 0                   # 0: no rotation
    rot_base: float = 10000.0
    chunk: Optional[int] = None         # mask.size
    v_mix: bool = False
    type: str = ATTENTION_TYPE


@dataclasses.dataclass(frozen=True)
class DenseConfig:
    ff: int
    kind: str = "dense"


@dataclasses.dataclass(frozen=True)
class MoeConfig:
    experts: int
    top: int
    expert_ff: int
    groups: int = 1
    keep: int = 1
    scale: float = 1.0
    shared_ff: int = 0
    kind: str = "moe"


@dataclasses.dataclass(frozen=True)
class LayerConfig:
    mixer: MixerConfig
    mlp: Optional[object]

    @property
    def type(self) -> str:
        return self.mixer.type


@dataclasses.dataclass(frozen=True)
class BurolornConfig:
    vocab: int
    width: int
    layers: Tuple[LayerConfig, ...]
    norm_eps: float
    logit_scale: float = 1.0
    side_dim: Optional[int] = None
    architecture: str = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def first_value_mix_layer(self) -> Optional[int]:
        for i, layer in enumerate(self.layers):
            if layer.mixer.v_mix:
                return i
        return None

    # -- json --------------------------------------------------------------
    @classmethod
    def from_json(cls, j: dict) -> "BurolornConfig":
        vocab, width = _get(j, "vocab", "top", int), _get(j, "width", "top", int)
        eps = _get(j.get("norm"), "eps", "norm", float)
        if eps <= 0:
            raise ModelConfigInvalid("config.json: norm.eps must be > 0")
        raw = j.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ModelConfigInvalid("config.json: 'layers' must be a list with at least one layer")
        layers = []
        first_mix = None
        for i, lj in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(lj, dict) or "type" not in lj or "mixer" not in lj or "mlp" not in lj:
                raise ModelConfigInvalid(f"config.json: {where} needs 'type', 'mixer' and 'mlp' (null for none)")
            if lj["type"] != ATTENTION_TYPE:
                raise ModelConfigInvalid(f"config.json: {where}.type {lj['type']!r} is not {ATTENTION_TYPE!r}")
            mj, mw = lj["mixer"], where + ".mixer"
            heads, kv_heads = _get(mj, "heads", mw, int), _get(mj, "kv_heads", mw, int)
            dim, vdim = _get(mj, "dim", mw, int), _get(mj, "vdim", mw, int)
            if heads % kv_heads:
                raise ModelConfigInvalid(f"config.json: {mw}: {heads} heads are not a multiple of {kv_heads} kv_heads")
            conv = _get(mj, "conv", mw, int) if mj.get("conv") not in (None, 0) else 0
            rot_dims, rot_base = 0, 10000.0
            if mj.get("rot") is not None:
                rot_dims, rot_base = _get(mj["rot"], "dims", mw + ".rot", int), _get(mj["rot"], "base", mw + ".rot", float)
                if rot_dims % 2 or rot_dims > dim or rot_base <= 0:
                    raise ModelConfigInvalid(f"config.json: {mw}.rot: dims must be even and at most dim, base > 0")
            chunk = _get(mj["mask"], "size", mw + ".mask", int) if mj.get("mask") is not None else None
            v_mix = mj.get("v_mix", False)
            if not isinstance(v_mix, bool):
                raise ModelConfigInvalid(f"config.json: {mw}.v_mix must be true or false")
            mixer = MixerConfig(heads, kv_heads, dim, vdim, _get(mj, "scale", mw, float), conv, rot_dims, rot_base,
                                chunk, v_mix)
            if v_mix:
                if first_mix is None:
                    first_mix = mixer
                elif (mixer.kv_heads, mixer.vdim) != (first_mix.kv_heads, first_mix.vdim):
                    raise ModelConfigInvalid(f"config.json: {mw}: values of {mixer.kv_heads} x {mixer.vdim} cannot be "
                                             f"mixed with the first such layer's {first_mix.kv_heads} x {first_mix.vdim}")
            mlp = None
            if lj["mlp"] is not None:
                pj, pw = lj["mlp"], where + ".mlp"
                kind = pj.get("kind") if isinstance(pj, dict) else None
                if kind == "dense":
                    mlp = DenseConfig(_get(pj, "ff", pw, int))
                elif kind == "moe":
                    rj = pj.get("router")
                    experts, top = _get(rj, "experts", pw + ".router", int), _get(rj, "top", pw + ".router", int)
                    groups = keep = 1
                    if rj.get("groups") is not None:
                        groups = _get(rj["groups"], "count", pw + ".router.groups", int)
                        keep = _get(rj["groups"], "keep", pw + ".router.groups", int)
                    if experts % groups or keep > groups or top > (experts // groups) * keep:
                        raise ModelConfigInvalid(f"config.json: {pw}.router: {experts} experts in {groups} groups of "
                                                 f"which {keep} are kept cannot give {top}")
                    scale = _get(rj, "scale", pw + ".router", float) if rj.get("scale") is not None else 1.0
                    shared = _get(pj["shared"], "ff", pw + ".shared", int) if pj.get("shared") is not None else 0
                    mlp = MoeConfig(experts, top, _get(pj.get("expert"), "ff", pw + ".expert", int), groups, keep,
                                    scale, shared)
                else:
                    raise ModelConfigInvalid(f"config.json: {pw}.kind must be 'dense' or 'moe'")
            layers.append(LayerConfig(mixer, mlp))
        logit_scale = _get(j, "logit_scale", "top", float) if j.get("logit_scale") is not None else 1.0
        side = _get(j["token_side"], "dim", "token_side", int) if j.get("token_side") is not None else None
        return cls(vocab, width, tuple(layers), eps, logit_scale, side)

    def to_json(self) -> dict:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            mj = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                  "v_mix": m.v_mix}
            if m.conv:
                mj["conv"] = m.conv
            if m.rot_dims:
                mj["rot"] = {"dims": m.rot_dims, "base": m.rot_base}
            if m.chunk is not None:
                mj["mask"] = {"size": m.chunk}
            mlp = None
            p = layer.mlp
            if isinstance(p, DenseConfig):
                mlp = {"kind": "dense", "ff": p.ff}
            elif p is not None:
                mlp = {"kind": "moe", "expert": {"ff": p.expert_ff},
                       "router": {"experts": p.experts, "top": p.top, "scale": p.scale,
                                  "groups": {"count": p.groups, "keep": p.keep}}}
                if p.shared_ff:
                    mlp["shared"] = {"ff": p.shared_ff}
            layers.append({"type": m.type, "mixer": mj, "mlp": mlp})
        j = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale, "layers": layers}
        if self.side_dim is not None:
            j["token_side"] = {"dim": self.side_dim}
        return j
