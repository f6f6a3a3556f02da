"""Gated delta rule with one decay per head and key channel: a linear-attention mixer with a state.

Per head, with S [key channels, value channels] starting at zero and carried from token to token:

    S <- diag(g_t) S
    u_t = beta_t (v_t - S^T k_t)
    S <- S + k_t u_t^T
    o_t = S^T q_t                      (the read-out sees the write of its own token)

q = x Wq^T and k = x Wk^T have ``kv_heads`` heads of ``key_dim`` (value head h reads head
h // (heads / kv_heads)), v = x Wv^T has ``heads`` heads of ``value_dim``.  Each of q, k, v passes a causal
convolution over time per channel (``taps`` taps, the last one the current token's, zeros before the start)
and silu; q and k are then unit vectors per head, x / sqrt(sum x^2 + 1e-6), q times key_dim^-1/2.
beta = sigmoid(x Wb^T) per head; g = exp(-exp(A_log[h]) softplus((x Wa1^T) Wa2^T + dt_bias)) per head and key
channel.  The output is o / rms(o) (per head, over value_dim) * norm_w * sigmoid((x Wg1^T) Wg2^T), then Wo.

What a request keeps between steps: S in float and the last ``taps - 1`` rows of q | k | v before the
convolution.  Everything after the projections is computed in float by the kernels of ``csrc/delta_rule.cu``.

The projections of x are three products: q | k | v | b in one merged matrix, the two narrow first stages
a1 | g1 in another, and the second stages a2 and g2 on the halves of that one's result.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import Unsupported
from .base import Mixer, StateNeed, TensorSpec

UNIT_EPS = 1e-6   # inside the root of the unit norms of q and k


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class ChannelGatedDelta(Mixer):
    kernel_groups = ("recurrent",)
    def __init__(self, hidden: int, heads: int, kv_heads: int, key_dim: int, value_dim: int, taps: int,
                 norm_eps: float, names: dict):
        """``names``: tensor names under the keys q, k, v, o, q_conv, k_conv, v_conv, b, A_log, dt_bias, a1, a2,
        g1, g2, norm.  The ranks of the two narrow pairs are read from the tensors' shapes by whoever builds
        the model and given as ``names["a_rank"]``, ``names["g_rank"]``."""
        if heads % kv_heads:
            raise Unsupported(f"{heads} heads are not a multiple of {kv_heads} q/k heads")
        if key_dim > 256:
            raise Unsupported(f"key size {key_dim}: the recurrence kernel holds up to 256 key channels per column")
        if taps < 1:
            raise Unsupported("a convolution has at least one tap")
        self.hidden, self.H, self.G, self.dk, self.dv = int(hidden), int(heads), int(kv_heads), int(key_dim), int(value_dim)
        self.taps, self.eps = int(taps), float(norm_eps)
        self.names = dict(names)
        self.a_rank, self.g_rank = int(self.names.pop("a_rank")), int(self.names.pop("g_rank"))
        self.qk_width, self.v_width = self.G * self.dk, self.H * self.dv
        # columns of the first product: q | k | v | b, each start a multiple of 8 (16 bytes in bfloat16)
        self.oq = 0
        self.ok = _pad8(self.qk_width)
        self.ov = self.ok + _pad8(self.qk_width)
        self.ob = self.ov + _pad8(self.v_width)
        self.proj_width = self.ob + _pad8(self.H)
        self.og1 = _pad8(self.a_rank)
        self.low_width = self.og1 + _pad8(self.g_rank)
        self.oga = _pad8(self.H * self.dk)
        self.ag_width = self.oga + _pad8(self.v_width)
        self.rt = None

    def tensor_specs(self):
        n, D = self.names, self.hidden
        C = self.qk_width
        return [TensorSpec(n["q"], (C, D)), TensorSpec(n["k"], (C, D)), TensorSpec(n["v"], (self.v_width, D)),
                TensorSpec(n["q_conv"], (C, self.taps), role="vector"),
                TensorSpec(n["k_conv"], (C, self.taps), role="vector"),
                TensorSpec(n["v_conv"], (self.v_width, self.taps), role="vector"),
                TensorSpec(n["b"], (self.H, D)),
                TensorSpec(n["A_log"], (self.H,), role="vector"),
                TensorSpec(n["dt_bias"], (self.H * self.dk,), role="vector"),
                TensorSpec(n["a1"], (self.a_rank, D)), TensorSpec(n["a2"], (self.H * self.dk, self.a_rank)),
                TensorSpec(n["g1"], (self.g_rank, D)), TensorSpec(n["g2"], (self.v_width, self.g_rank)),
                TensorSpec(n["norm"], (self.dv,), role="vector", init="one_plus_normal"),
                TensorSpec(n["o"], (D, self.v_width))]

    def state_need(self):
        C = 2 * self.qk_width + self.v_width
        return [StateNeed((self.H, self.dv, self.dk), torch.float32, "S"),
                StateNeed((max(self.taps - 1, 1), C), None, "conv")]

    def bind(self, rt, fetch):
        self.rt = rt
        n, D = self.names, self.hidden

        def stacked(width, pieces):
            w = torch.zeros((width, pieces[0][1].shape[1]), dtype=rt.dtype, device=rt.device)
            for off, t in pieces:
                w[off:off + t.shape[0]] = t
            return w

        self.w_proj = stacked(self.proj_width, [(self.oq, fetch(n["q"])), (self.ok, fetch(n["k"])),
                                                (self.ov, fetch(n["v"])), (self.ob, fetch(n["b"]))])
        self.w_low = stacked(self.low_width, [(0, fetch(n["a1"])), (self.og1, fetch(n["g1"]))])
        # the second stages read a slice of the narrow product's rows: columns up to a multiple of 8, the
        # added ones zero on both sides
        a2, g2 = fetch(n["a2"]), fetch(n["g2"])
        self.w_a2 = torch.zeros((self.H * self.dk, _pad8(self.a_rank)), dtype=rt.dtype, device=rt.device)
        self.w_a2[:, :self.a_rank] = a2
        self.w_g2 = torch.zeros((self.v_width, _pad8(self.g_rank)), dtype=rt.dtype, device=rt.device)
        self.w_g2[:, :self.g_rank] = g2
        # tap-major: the kernel reads the weights of neighbouring channels of one tap together
        self.conv_w = torch.cat([fetch(n["q_conv"]), fetch(n["k_conv"]), fetch(n["v_conv"])], dim=0).float().t().contiguous()
        self.A_log = fetch(n["A_log"]).float().contiguous()
        self.dt_bias = fetch(n["dt_bias"]).float().contiguous()
        self.norm_w = fetch(n["norm"]).float().contiguous()
        self.w_o = fetch(n["o"])

    def forward(self, x, step, cache, state):
        rt = self.rt
        x = rt.rows(x)
        T = x.shape[0]
        G, H, dk, dv = self.G, self.H, self.dk, self.dv
        f32 = torch.float32
        proj = rt.scratch.get("delta_proj", (rt.max_tokens, self.proj_width), rt.dtype)[:T]
        rt.linear(proj, x, self.w_proj)
        low = rt.scratch.get("delta_low", (rt.max_tokens, self.low_width), rt.dtype)[:T]
        rt.linear(low, x, self.w_low)
        ag = rt.scratch.get("delta_ag", (rt.max_tokens, self.ag_width), rt.dtype)[:T]
        rt.linear(ag[:, :H * dk], low[:, :self.og1], self.w_a2)
        rt.linear(ag[:, self.oga:self.oga + self.v_width], low[:, self.og1:], self.w_g2)
        qn = rt.scratch.get("delta_q", (rt.max_tokens, G, dk), f32)[:T]
        kn = rt.scratch.get("delta_k", (rt.max_tokens, G, dk), f32)[:T]
        vv = rt.scratch.get("delta_v", (rt.max_tokens, H, dv), f32)[:T]
        gg = rt.scratch.get("delta_g", (rt.max_tokens, H, dk), f32)[:T]
        bb = rt.scratch.get("delta_beta", (rt.max_tokens, H), f32)[:T]
        offsets = (self.oq, self.ok, self.ov, self.ob)
        S, conv = state["S"], state["conv"]
        kernels.delta_prepare(proj, offsets, ag, self.conv_w, self.taps, conv, self.A_log, self.dt_bias,
                              step.entry_of_token, step.cu_q, step.state_slot, qn, kn, vv, gg, bb, G, H, dk, dv,
                              dk ** -0.5, UNIT_EPS)
        kernels.conv_state_update(proj, offsets, conv, self.taps, step.cu_q, step.state_slot, step.n_entries,
                                  G, H, dk, dv)
        o = rt.scratch.get("delta_o", (rt.max_tokens, H, dv), f32)[:T]
        kernels.delta_recurrence(qn, kn, vv, gg, bb, S, o, step.cu_q, step.state_slot, step.n_entries, G, H, dk, dv)
        y = rt.scratch.get("delta_y", (rt.max_tokens, self.v_width), rt.dtype)[:T]
        kernels.gated_head_rmsnorm(y, o, ag[:, self.oga:], self.norm_w, H, dv, self.eps)
        out = rt.scratch.get(self.out_key, (rt.max_tokens, self.hidden), rt.dtype)[:T]
        return rt.linear(out, y, self.w_o)
