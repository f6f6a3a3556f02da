"""Typed configuration of Gevovik, a decoder whose config.json lists its layers one by one.

    {"architecture": "Gevovik", "vocab": V, "width": D, "norm": {"eps": e},
     "embedding": {"scale": s, "bigram": {"buckets": n, "mul_prev": a, "mul_cur": b}},      (bigram optional)
     "layers": [{"type": T, "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}, ...]}

Mixer types and their keys:

* ``mamba2``: heads, vdim (channels per head), state, groups, conv (taps), norm_groups.
* ``parallel``: left_scale, right_scale and a pair of mixers that run on the same input,
  ``left`` {heads, kv_heads, dim, vdim, scale, ``rot`` {dims, base, ``scaling`` {factor, original, fast, slow}},
  ``mask`` {size}}: softmax attention over a window whose heads' scores are mixed before the softmax, and
  ``right`` {heads, kv_heads, dim, vdim, conv}: the gated delta rule with a decay per key channel.  The ranks of
  the delta rule's two narrow projection pairs are no keys of the file: they are the shapes of the tensors
  ``l<i>.mix.right.a1`` and ``.g1`` (``with_shapes``); a configuration made in code carries them as ``a_rank`` and
  ``g_rank`` and writes them out under these names.
* ``latent_attention``: heads, dim, rot_dim, vdim, kv_rank, scale, ``rot`` {dims, base}, and optionally
  ``kv_from``: the layer whose cached rows this one reads instead of making its own.

``rot``, ``rot.scaling`` and ``mask`` are taken where they are present.  Nothing here is a default for a size: a
missing key is an error.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Tuple

from ..errors import ModelConfigInvalid
from .tugelorn import _get

ARCHITECTURE = "Gevovik"
SSM_TYPE = "mamba2"
PARALLEL_TYPE = "parallel"
LATENT_TYPE = "latent_attention"


@dataclasses.dataclass(frozen=True)
class RampScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclasses.dataclass(frozen=True)
class Rotation:
    dims: int
    base: float
    scaling: Optional[RampScaling] = None


@dataclasses.dataclass(frozen=True)
class SsmMixerConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int
    type: str = SSM_TYPE


@dataclasses.dataclass(frozen=True)
class TalkingAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[Rotation] = None
    window: Optional[int] = None


@dataclasses.dataclass(frozen=True)
class DeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    a_rank: Optional[int] = None
    g_rank: Optional[int] = None


@dataclasses.dataclass(frozen=True)
class ParallelMixerConfig:
    left: TalkingAttentionConfig
    right: DeltaConfig
    left_scale: float
    right_scale: float
    type: str = PARALLEL_TYPE


@dataclasses.dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: Rotation
    kv_from: Optional[int] = None
    type: str = LATENT_TYPE


@dataclasses.dataclass(frozen=True)
class MlpConfig:
    ff: int
    kind: str = "dense"


@dataclasses.dataclass(frozen=True)
class LayerConfig:
    mixer: object
    mlp: Optional[MlpConfig]

    @property
    def type(self) -> str:
        return self.mixer.type


@dataclasses.dataclass(frozen=True)
class PairTable:
    buckets: int
    mul_prev: int
    mul_cur: int


def _rotation(rj, where, limit, what) -> Rotation:
    scaling = None
    if rj.get("scaling") is not None:
        sj, sw = rj["scaling"], where + ".scaling"
        scaling = RampScaling(*(_get(sj, k, sw, float) for k in ("factor", "original", "fast", "slow")))
        if min(scaling.factor, scaling.original, scaling.fast, scaling.slow) <= 0:
            raise ModelConfigInvalid(f"config.json: {sw}: factor, original, fast and slow must be > 0")
    rot = Rotation(_get(rj, "dims", where, int), _get(rj, "base", where, float), scaling)
    if rot.dims % 2 or rot.dims > limit or rot.base <= 1:
        raise ModelConfigInvalid(f"config.json: {where}: dims must be even and at most {what}, base > 1")
    return rot


def _rotation_json(rot: Rotation) -> dict:
    j = {"dims": rot.dims, "base": rot.base}
    if rot.scaling is not None:
        s = rot.scaling
        j["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
    return j


@dataclasses.dataclass(frozen=True)
class GevovikConfig:
    vocab: int
    width: int
    layers: Tuple[LayerConfig, ...]
    norm_eps: float
    embed_scale: float
    pair: Optional[PairTable] = None
    architecture: str = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def with_shapes(self, shapes: dict) -> "GevovikConfig":
        """The sizes that only the tensors give (a checkpoint's name -> shape), filled in."""
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if m.type == PARALLEL_TYPE and (m.right.a_rank is None or m.right.g_rank is None):
                try:
                    a, g = shapes[f"l{i}.mix.right.a1"], shapes[f"l{i}.mix.right.g1"]
                    right = dataclasses.replace(m.right, a_rank=int(a[0]), g_rank=int(g[0]))
                except (KeyError, IndexError, TypeError):
                    raise ModelConfigInvalid(f"layer {i}: the ranks of right.a1 and right.g1 are neither in "
                                             f"config.json nor tensors of the checkpoint") from None
                layer = dataclasses.replace(layer, mixer=dataclasses.replace(m, right=right))
            layers.append(layer)
        return dataclasses.replace(self, layers=tuple(layers))

    # -- json --------------------------------------------------------------
    @classmethod
    def from_json(cls, j: dict) -> "GevovikConfig":
        vocab, width = _get(j, "vocab", "top", int), _get(j, "width", "top", int)
        eps = _get(j.get("norm"), "eps", "norm", float)
        if eps <= 0:
            raise ModelConfigInvalid("config.json: norm.eps must be > 0")
        ej = j.get("embedding")
        scale = _get(ej, "scale", "embedding", float)
        pair = None
        if ej.get("bigram") is not None:
            bj = ej["bigram"]
            pair = PairTable(*(_get(bj, k, "embedding.bigram", int) for k in ("buckets", "mul_prev", "mul_cur")))
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
            if t == SSM_TYPE:
                mixer = SsmMixerConfig(*(_get(mj, k, mw, int) for k in ("heads", "vdim", "state", "groups", "conv",
                                                                        "norm_groups")))
                if mixer.heads % mixer.groups or (mixer.heads * mixer.vdim) % mixer.norm_groups:
                    raise ModelConfigInvalid(f"config.json: {mw}: heads must be a multiple of groups, and heads * vdim "
                                             f"of norm_groups")
            elif t == PARALLEL_TYPE:
                lw, rw = mw + ".left", mw + ".right"
                lm, rm = mj.get("left"), mj.get("right")
                heads, kv = _get(lm, "heads", lw, int), _get(lm, "kv_heads", lw, int)
                dim = _get(lm, "dim", lw, int)
                rot = _rotation(lm["rot"], lw + ".rot", dim, "dim") if lm.get("rot") is not None else None
                window = _get(lm["mask"], "size", lw + ".mask", int) if lm.get("mask") is not None else None
                left = TalkingAttentionConfig(heads, kv, dim, _get(lm, "vdim", lw, int), _get(lm, "scale", lw, float),
                                              rot, window)
                ranks = {k: (_get(rm, k, rw, int) if k in rm else None) for k in ("a_rank", "g_rank")}
                right = DeltaConfig(*(_get(rm, k, rw, int) for k in ("heads", "kv_heads", "dim", "vdim", "conv")),
                                    **ranks)
                if left.heads % left.kv_heads or right.heads % right.kv_heads:
                    raise ModelConfigInvalid(f"config.json: {mw}: heads must be a multiple of kv_heads on both sides")
                mixer = ParallelMixerConfig(left, right, _get(mj, "left_scale", mw, float),
                                            _get(mj, "right_scale", mw, float))
            elif t == LATENT_TYPE:
                rot_dim = _get(mj, "rot_dim", mw, int)
                kv_from = None
                if mj.get("kv_from") is not None:
                    kv_from = mj["kv_from"]
                    if isinstance(kv_from, bool) or not isinstance(kv_from, int) or not (0 <= kv_from < i):
                        raise ModelConfigInvalid(f"config.json: {mw}.kv_from must name an earlier layer")
                mixer = LatentMixerConfig(_get(mj, "heads", mw, int), _get(mj, "dim", mw, int), rot_dim,
                                          _get(mj, "vdim", mw, int), _get(mj, "kv_rank", mw, int),
                                          _get(mj, "scale", mw, float),
                                          _rotation(mj.get("rot") or {}, mw + ".rot", rot_dim, "rot_dim"), kv_from)
                if kv_from is not None:
                    src = layers[kv_from].mixer
                    if (src.type != LATENT_TYPE or src.kv_from is not None or src.kv_rank != mixer.kv_rank
                            or src.rot_dim != mixer.rot_dim or src.rot != mixer.rot):
                        raise ModelConfigInvalid(f"config.json: {mw}.kv_from: layer {kv_from} must be a latent "
                                                 f"attention layer with rows of its own and the same kv_rank, "
                                                 f"rot_dim and rot")
            else:
                raise ModelConfigInvalid(f"config.json: {where}.type {t!r} is not one of "
                                         f"{(SSM_TYPE, PARALLEL_TYPE, LATENT_TYPE)}")
            mlp = None
            if lj["mlp"] is not None:
                pj = lj["mlp"]
                if not isinstance(pj, dict) or pj.get("kind") != "dense":
                    raise ModelConfigInvalid(f"config.json: {where}.mlp.kind must be 'dense'")
                mlp = MlpConfig(_get(pj, "ff", where + ".mlp", int))
            layers.append(LayerConfig(mixer, mlp))
        return cls(vocab, width, tuple(layers), eps, scale, pair)

    def to_json(self) -> dict:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if m.type == SSM_TYPE:
                mj = {"heads": m.heads, "vdim": m.vdim, "state": m.state, "groups": m.groups, "conv": m.conv,
                      "norm_groups": m.norm_groups}
            elif m.type == PARALLEL_TYPE:
                a, d = m.left, m.right
                lj = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
                if a.rot is not None:
                    lj["rot"] = _rotation_json(a.rot)
                if a.window is not None:
                    lj["mask"] = {"size": a.window}
                rj = {"heads": d.heads, "kv_heads": d.kv_heads, "dim": d.dim, "vdim": d.vdim, "conv": d.conv}
                if d.a_rank is not None:
                    rj["a_rank"], rj["g_rank"] = d.a_rank, d.g_rank
                mj = {"left": lj, "right": rj, "left_scale": m.left_scale, "right_scale": m.right_scale}
            else:
                mj = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                      "scale": m.scale, "rot": _rotation_json(m.rot)}
                if m.kv_from is not None:
                    mj["kv_from"] = m.kv_from
            mlp = None if layer.mlp is None else {"kind": layer.mlp.kind, "ff": layer.mlp.ff}
            layers.append({"type": m.type, "mixer": mj, "mlp": mlp})
        ej = {"scale": self.embed_scale}
        if self.pair is not None:
            ej["bigram"] = {"buckets": self.pair.buckets, "mul_prev": self.pair.mul_prev, "mul_cur": self.pair.mul_cur}
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "embedding": ej, "layers": layers}
