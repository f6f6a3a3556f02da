"""Gevovik put together from the parts: state space layers, pairs of an attention and a delta rule on the same input, and
latent attention layers that may read an earlier layer's cached rows.

A layer is a ``PostNormBlock``: h += norm1(mixer(h)); h += norm2(ff(h)), the sublayers reading the stream itself and
each norm an RMS norm whose weight is a single scalar.  The mixers: ``SelectiveStateSpace``; ``ParallelMixers`` of a
``GroupedQueryAttention`` over a window (head norms, a rotation whose slow pairs are stretched, scores times a number
per head and mixed over the heads before the softmax, a gate per head) and a ``ChannelGatedDelta``;
``LatentAttention`` over every earlier token with a sink, rotated in interleaved pairs, optionally without rows of
its own (``RunEntry.cache_of``).  The feed-forward is ``SquaredReLU``.  The embedding is the token's row times a
constant plus a row of a second table chosen by the pair (previous token, token).

Tensor names: ``embed``, ``bigram``, ``l<i>.norm1 / norm2``, ``l<i>.mix.*`` (``.left.*`` and ``.right.*`` in a
pair), ``l<i>.mlp.up / down``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.gevovik import LATENT_TYPE, PARALLEL_TYPE, SSM_TYPE, GevovikConfig
from ..engine.plan import ModelPlan, RunEntry
from ..errors import ModelConfigInvalid
from ..parts import (ChannelGatedDelta, GroupedQueryAttention, LatentAttention, OutputHead, ParallelMixers,
                     PostNormBlock, RMSNorm, RotaryHalf, SelectiveStateSpace, SquaredReLU, TokenEmbedding)
from ..parts.position import NoPosition


def _ssm(cfg: GevovikConfig, m, p: str):
    names = {"in": p + "in", "conv": p + "conv", "conv_bias": p + "conv.b", "dt_bias": p + "dt_bias",
             "A_log": p + "A_log", "D": p + "D", "norm": p + "norm", "o": p + "o"}
    return SelectiveStateSpace(cfg.width, m.heads, m.vdim, m.state, m.groups, m.conv, m.norm_groups, cfg.norm_eps, names)


def _talking_attention(cfg: GevovikConfig, m, p: str):
    hd = GroupedQueryAttention.kernel_head_dim(m.dim, m.vdim)
    position = NoPosition()
    if m.rot is not None:
        sc = m.rot.scaling
        ramp = None if sc is None else {"factor": sc.factor, "original": sc.original, "fast": sc.fast, "slow": sc.slow}
        position = RotaryHalf(hd, m.rot.base, rotary_dim=m.rot.dims, ramp_scaling=ramp,
                              linear_scaling=None if ramp is not None else 1.0)
    names = {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o", "q_norm": p + "q.norm", "k_norm": p + "k.norm",
             "talk": p + "talk", "temp": p + "temp", "gate": p + "g"}
    return GroupedQueryAttention(hidden=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
                                 position=position, names=names, qk_norm_eps=cfg.norm_eps, window=m.window,
                                 scale=m.scale, value_dim=m.vdim)


def _delta(cfg: GevovikConfig, m, p: str, layer: int):
    if m.a_rank is None or m.g_rank is None:
        raise ModelConfigInvalid(f"layer {layer}: the ranks of the delta rule's narrow projections are unknown "
                                 f"(GevovikConfig.with_shapes fills them in from a checkpoint)")
    names = {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o", "q_conv": p + "q.conv", "k_conv": p + "k.conv",
             "v_conv": p + "v.conv", "b": p + "b", "A_log": p + "A_log", "dt_bias": p + "dt_bias", "a1": p + "a1",
             "a2": p + "a2", "g1": p + "g1", "g2": p + "g2", "norm": p + "norm", "a_rank": m.a_rank,
             "g_rank": m.g_rank}
    return ChannelGatedDelta(cfg.width, m.heads, m.kv_heads, m.dim, m.vdim, m.conv, cfg.norm_eps, names)


def _latent(cfg: GevovikConfig, m, p: str):
    names = {"q": p + "q", "dkv": p + "dkv", "dkv_norm": p + "dkv.norm", "uk": p + "uk", "uv": p + "uv",
             "sink": p + "sink", "o": p + "o"}
    return LatentAttention(cfg.width, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, None, m.scale, m.rot.base,
                           m.rot.dims, cfg.norm_eps, names, interleaved=True, own_kv=m.kv_from is None)


def build_plan(cfg: GevovikConfig) -> ModelPlan:
    D, eps = cfg.width, cfg.norm_eps
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        cache_of = None
        if m.type == SSM_TYPE:
            mixer = _ssm(cfg, m, p + "mix.")
        elif m.type == PARALLEL_TYPE:
            mixer = ParallelMixers(D, _talking_attention(cfg, m.left, p + "mix.left."),
                                   _delta(cfg, m.right, p + "mix.right.", i), m.left_scale, m.right_scale)
        elif m.type == LATENT_TYPE:
            mixer = _latent(cfg, m, p + "mix.")
            cache_of = m.kv_from     # (no layer runs twice: a layer's number is its place in the order)
        else:
            raise ModelConfigInvalid(f"layer {i}: mixer type {m.type!r}")
        ffn = post2 = None
        if layer.mlp is not None:
            ffn = SquaredReLU(D, layer.mlp.ff, {"up": p + "mlp.up", "down": p + "mlp.down"})
            post2 = RMSNorm(D, eps, p + "norm2", scalar=True)
        layers.append(PostNormBlock(D, mixer, RMSNorm(D, eps, p + "norm1", scalar=True), ffn, post2))
        order.append(RunEntry(i, cache_of=cache_of))
    pair = None
    if cfg.pair is not None:
        pair = {"name": "bigram", "buckets": cfg.pair.buckets, "mul_prev": cfg.pair.mul_prev,
                "mul_cur": cfg.pair.mul_cur}
    return ModelPlan(embedding=TokenEmbedding(cfg.vocab, D, "embed", scale=cfg.embed_scale, pair=pair), layers=layers,
                     order=order, final_norm=RMSNorm(D, eps, "final.norm", scalar=True),
                     head=OutputHead(D, cfg.vocab, "head"), vocab_size=cfg.vocab, max_position=None)
