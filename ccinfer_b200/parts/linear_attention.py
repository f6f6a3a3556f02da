"""Gated linear attention: a linear-attention mixer with one decay per head and key channel, and a state.

Per head, with S [key channels, value channels] starting at zero and carried from token to token:

    S <- diag(alpha_t) S + k_t v_t^T;    o_t = S^T q_t

q = Wq x * dim^-1/2, k = Wk x (heads x dim), v = Wv x (heads x vdim); alpha = sigmoid(z)^(1 / tau) with
z = Wa2 (Wa1 x) + b per head and key channel.  Each head's o is RMS-normed over vdim (one weight vector for all
heads), the heads are multiplied by silu(Wg x) and projected by Wo.

What a request keeps between steps is S in float.  Everything after the projections is float (kernels of
``csrc/linear_attention.cu`` and the plain form of the recurrence in ``csrc/delta_rule.cu``).  q, k, v, the gate
and the narrow first stage of the decay are ONE merged product of x.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import Unsupported
from .base import Mixer, StateNeed, TensorSpec


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class GatedLinearAttention(Mixer):
    kernel_groups = ("recurrent",)
    def __init__(self, hidden: int, heads: int, key_dim: int, value_dim: int, tau: float, decay_rank: int,
                 norm_eps: float, names: dict):
        """``names``: tensor names under the keys q, k, v, g, o, norm, a1, a2, a2_bias."""
        if key_dim > 256:
            raise Unsupported(f"key size {key_dim}: the recurrence kernel holds up to 256 key channels per column")
        if not tau > 0:
            raise Unsupported("tau must be > 0")
        self.hidden, self.H, self.dk, self.dv = int(hidden), int(heads), int(key_dim), int(value_dim)
        self.tau, self.rank, self.eps = float(tau), int(decay_rank), float(norm_eps)
        self.names = dict(names)
        qk, vw = self.H * self.dk, self.H * self.dv
        self.oq = 0
        self.ok = _pad8(qk)
        self.ov = self.ok + _pad8(qk)
        self.og = self.ov + _pad8(vw)
        self.oa = self.og + _pad8(vw)
        self.in_width = self.oa + _pad8(self.rank)
        self.rt = None

    def tensor_specs(self):
        n, D = self.names, self.hidden
        qk, vw = self.H * self.dk, self.H * self.dv
        return [TensorSpec(n["q"], (qk, D)), TensorSpec(n["k"], (qk, D)), TensorSpec(n["v"], (vw, D)),
                TensorSpec(n["g"], (vw, D)), TensorSpec(n["o"], (D, vw)),
                TensorSpec(n["norm"], (self.dv,), role="vector", init="one_plus_normal"),
                TensorSpec(n["a1"], (self.rank, D)), TensorSpec(n["a2"], (qk, self.rank)),
                TensorSpec(n["a2_bias"], (qk,), role="vector")]

    def state_need(self):
        return StateNeed((self.H, self.dv, self.dk), torch.float32, "S")

    def bind(self, rt, fetch):
        self.rt = rt
        n = self.names
        w = torch.zeros((self.in_width, self.hidden), dtype=rt.dtype, device=rt.device)
        for off, name in ((self.oq, "q"), (self.ok, "k"), (self.ov, "v"), (self.og, "g"), (self.oa, "a1")):
            t = fetch(n[name])
            w[off:off + t.shape[0]] = t
        self.w_in = w
        # the second stage reads a slice of the merged product's rows: columns up to a multiple of 8, the added
        # ones zero on both sides
        a2 = fetch(n["a2"])
        self.w_a2 = torch.zeros((a2.shape[0], _pad8(self.rank)), dtype=rt.dtype, device=rt.device)
        self.w_a2[:, :self.rank] = a2
        self.a2_bias = fetch(n["a2_bias"]).float().contiguous()
        self.norm_w = fetch(n["norm"]).float().contiguous()
        self.w_o = fetch(n["o"])

    def forward(self, x, step, cache, state):
        rt = self.rt
        x = rt.rows(x)
        T = x.shape[0]
        H, dk, dv = self.H, self.dk, self.dv
        f32 = torch.float32
        proj = rt.scratch.get("gla_proj", (rt.max_tokens, self.in_width), rt.dtype)[:T]
        rt.linear(proj, x, self.w_in)
        a = rt.scratch.get("gla_decay", (rt.max_tokens, H * dk), rt.dtype)[:T]
        rt.linear(a, proj[:, self.oa:self.oa + self.w_a2.shape[1]], self.w_a2)
        qn = rt.scratch.get("delta_q", (rt.max_tokens, H, dk), f32)[:T]
        kn = rt.scratch.get("delta_k", (rt.max_tokens, H, dk), f32)[:T]
        vv = rt.scratch.get("delta_v", (rt.max_tokens, H, dv), f32)[:T]
        gg = rt.scratch.get("delta_g", (rt.max_tokens, H, dk), f32)[:T]
        kernels.gla_prepare(proj, (self.oq, self.ok, self.ov), a, self.a2_bias, qn, kn, vv, gg, H, dk, dv,
                            dk ** -0.5, self.tau)
        o = rt.scratch.get("delta_o", (rt.max_tokens, H, dv), f32)[:T]
        kernels.gated_linear_recurrence(qn, kn, vv, gg, state, o, step.cu_q, step.state_slot, step.n_entries, H, dk, dv)
        y = rt.scratch.get("delta_y", (rt.max_tokens, H * dv), rt.dtype)[:T]
        kernels.gated_head_rmsnorm(y, o, proj[:, self.og:], self.norm_w, H, dv, self.eps, silu_gate=True)
        out = rt.scratch.get(self.out_key, (rt.max_tokens, self.hidden), rt.dtype)[:T]
        return rt.linear(out, y, self.w_o)
