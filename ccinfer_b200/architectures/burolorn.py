"""Burolorn put together from the parts: attention layers with short convolutions on q, k and v, per-head norms,
a partial rotation, a chunked mask, a sink in the softmax, values mixed with the first layer's, a gate per head;
dense gated feed-forwards and mixtures of gated experts in any order; a per-layer token input; scaled logits.

A layer is a ``PreNormBlock``: h += mixer(norm1(h)); h += ff(norm2(h)); h += side(h, token), the norms plain RMS
norms.  The mixer is ``GroupedQueryAttention`` with its options; the mixture ``MixtureOfExperts`` with sigmoid
scores, a group's score the sum of its two best, renormalised weights times the router's scale, and a shared
expert behind a sigmoid gate per token.  The head is a matrix of its own; the logits' scale rides on the last
norm's weight.

Tensor names: ``embed``, ``side.embed``, ``l<i>.norm1 / norm2``, ``l<i>.mix.q / k / v / o / g / sink / vmix``,
``l<i>.mix.q.norm / k.norm``, ``l<i>.mix.q.conv / k.conv / v.conv``, ``l<i>.mlp.gate / up / down`` or
``l<i>.mlp.router / e<k>.gate / e<k>.up / e<k>.down / shared.gate / shared.up / shared.down / shared.sg``,
``l<i>.side.gate / proj / norm``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from .. import kernels
from ..config.burolorn import BurolornConfig, DenseConfig
from ..engine.plan import ModelPlan, RunEntry
from ..parts import (GroupedQueryAttention, MixtureOfExperts, NoPosition, OutputHead, PreNormBlock, RMSNorm,
                     RotaryHalf, SwiGLU, TokenEmbedding, TokenSideInput)

GROUP_SCORE_TOP = 2        # a group's score is the sum of its two largest scores
VALUE_MIX_KEY = "burolorn"


def _mixer(cfg: BurolornConfig, m, p: str, layer: int, first_mix):
    names = {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o", "q_norm": p + "q.norm", "k_norm": p + "k.norm",
             "sink": p + "sink", "gate": p + "g"}
    if m.conv:
        names.update({"q_conv": p + "q.conv", "k_conv": p + "k.conv", "v_conv": p + "v.conv"})
    value_mix = None
    if m.v_mix:
        names["vmix"] = p + "vmix"
        value_mix = ("first" if layer == first_mix else "mix", VALUE_MIX_KEY)
    hd = GroupedQueryAttention.kernel_head_dim(m.dim, m.vdim)
    # the angles' frequencies are base^(-2i / dims), evaluated in float64 and rounded once
    position = (RotaryHalf(hd, m.rot_base, rotary_dim=m.rot_dims, linear_scaling=1.0) if m.rot_dims else NoPosition())
    return GroupedQueryAttention(cfg.width, m.heads, m.kv_heads, m.dim, position, names, qk_norm_eps=cfg.norm_eps,
                                 scale=m.scale, value_dim=m.vdim, chunk=m.chunk, conv_taps=m.conv,
                                 value_mix=value_mix)


def _feed_forward(cfg: BurolornConfig, q, p: str):
    if isinstance(q, DenseConfig):
        return SwiGLU(cfg.width, q.ff, {"gate": p + "gate", "up": p + "up", "down": p + "down"})
    names = {"router": p + "router", "gate": p + "e{e}.gate", "up": p + "e{e}.up", "down": p + "e{e}.down",
             "shared_gate_proj": p + "shared.gate", "shared_up": p + "shared.up", "shared_down": p + "shared.down",
             "shared_gate": p + "shared.sg"}
    rule = kernels.RouteRule("sigmoid", GROUP_SCORE_TOP, renorm=True, scale=q.scale)
    return MixtureOfExperts(cfg.width, q.experts, q.top, q.expert_ff, names, q.groups, q.keep, q.shared_ff,
                            activation="swiglu", rule=rule)


def build_plan(cfg: BurolornConfig) -> ModelPlan:
    D, eps = cfg.width, cfg.norm_eps
    n_layers = len(cfg.layers)
    first_mix = cfg.first_value_mix_layer()
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        norm2 = ffn = None
        if layer.mlp is not None:
            norm2 = RMSNorm(D, eps, p + "norm2")
            ffn = _feed_forward(cfg, layer.mlp, p + "mlp.")
        side = None
        if cfg.side_dim is not None:
            side = TokenSideInput(cfg.vocab, D, cfg.side_dim, i * cfg.side_dim, n_layers * cfg.side_dim, eps,
                                  {"table": "side.embed", "gate": p + "side.gate", "proj": p + "side.proj",
                                   "norm": p + "side.norm"})
        layers.append(PreNormBlock(RMSNorm(D, eps, p + "norm1"), _mixer(cfg, layer.mixer, p + "mix.", i, first_mix),
                                   norm2, ffn, side))
    return ModelPlan(embedding=TokenEmbedding(cfg.vocab, D, "embed"), layers=layers,
                     order=[RunEntry(i) for i in range(n_layers)],
                     final_norm=RMSNorm(D, eps, "final.norm", weight_scale=cfg.logit_scale),
                     head=OutputHead(D, cfg.vocab, "head"), vocab_size=cfg.vocab, max_position=None)
