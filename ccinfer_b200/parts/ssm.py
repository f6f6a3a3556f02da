"""A selective state space mixer in the form of state-space duality, run as its recurrence.

With H heads of P channels (``inner`` = H P), a state of N channels per head and G groups of B and C:

    [z | x | B | C | dt] = Win h            z, x: inner;  B, C: G N;  dt: H
    x | B | C  <-  silu(conv(x | B | C) + bias)     per channel c: sum_j w[c, j] * u[t - (taps - 1) + j, c], inputs
                                                    from before the sequence began counting as 0
    dt = softplus(dt + dt_bias);   a = exp(-exp(A_log_h) dt)
    S <- a_t S + B_t (dt_t x_t)^T;   y_t = S^T C_t + D_h x_t       per head h, with the B and C of group h // (H / G)
    y <- slices(y * silu(z)) each over the root of its mean square (+ eps), times a weight per channel;   out = Wo y

There are ``norm_groups`` slices of equal size, and the gating by z is applied first, the norm second.  What a request keeps between steps: S [H, P, N] in float and the last
``taps - 1`` rows of x | B | C before the convolution.  Everything after the projection is float
(``csrc/ssm.cu``; the recurrence is the plain form of ``csrc/delta_rule.cu`` with one decay per head and a step
size on the write).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import Unsupported
from .base import Mixer, StateNeed, TensorSpec


class SelectiveStateSpace(Mixer):
    kernel_groups = ("recurrent",)
    def __init__(self, hidden: int, heads: int, head_dim: int, state: int, groups: int, taps: int, norm_groups: int,
                 norm_eps: float, names: dict):
        """``names``: tensor names under the keys in, conv, conv_bias, dt_bias, A_log, D, norm, o."""
        if heads % groups:
            raise Unsupported(f"{heads} heads are not a multiple of {groups} groups")
        if (heads * head_dim) % norm_groups:
            raise Unsupported(f"{heads * head_dim} inner channels do not split into {norm_groups} equal slices")
        if state > 256:
            raise Unsupported(f"state size {state}: the recurrence kernel holds up to 256 state channels per column")
        if taps < 1:
            raise Unsupported("a convolution has at least one tap")
        self.hidden, self.H, self.P, self.N, self.G = int(hidden), int(heads), int(head_dim), int(state), int(groups)
        self.taps, self.parts, self.eps = int(taps), int(norm_groups), float(norm_eps)
        self.names = dict(names)
        self.inner = self.H * self.P
        self.conv_width = self.inner + 2 * self.G * self.N
        self.in_width = 2 * self.inner + 2 * self.G * self.N + self.H
        self.proj_width = -(-self.in_width // 8) * 8   # rows of the projection's result start on 16 bytes
        self.rt = None

    def tensor_specs(self):
        n, D = self.names, self.hidden
        return [TensorSpec(n["in"], (self.in_width, D)),
                TensorSpec(n["conv"], (self.conv_width, self.taps), role="vector"),
                TensorSpec(n["conv_bias"], (self.conv_width,), role="vector"),
                TensorSpec(n["dt_bias"], (self.H,), role="vector"), TensorSpec(n["A_log"], (self.H,), role="vector"),
                TensorSpec(n["D"], (self.H,), role="vector", init="one_plus_normal"),
                TensorSpec(n["norm"], (self.inner,), role="vector", init="one_plus_normal"),
                TensorSpec(n["o"], (D, self.inner))]

    def state_need(self):
        return [StateNeed((self.H, self.P, self.N), torch.float32, "S"),
                StateNeed((max(self.taps - 1, 1), self.conv_width), None, "conv")]

    def bind(self, rt, fetch):
        self.rt = rt
        n = self.names
        self.w_in = fetch(n["in"])
        if self.proj_width != self.in_width:   # zero rows: columns that nobody reads
            w = torch.zeros((self.proj_width, self.hidden), dtype=self.w_in.dtype, device=self.w_in.device)
            w[:self.in_width] = self.w_in
            self.w_in = w
        self.conv_w = fetch(n["conv"]).float().t().contiguous()      # tap-major
        self.conv_b = fetch(n["conv_bias"]).float().contiguous()
        self.dt_bias = fetch(n["dt_bias"]).float().contiguous()
        self.A_log = fetch(n["A_log"]).float().contiguous()
        self.skip = fetch(n["D"]).float().contiguous()
        self.norm_w = fetch(n["norm"]).float().contiguous()
        self.w_o = fetch(n["o"])

    def forward(self, x, step, cache, state):
        rt = self.rt
        x = rt.rows(x)
        T = x.shape[0]
        H, P, N, G = self.H, self.P, self.N, self.G
        f32 = torch.float32
        proj = rt.scratch.get("ssm_proj", (rt.max_tokens, self.proj_width), rt.dtype)[:T]
        rt.linear(proj, x, self.w_in)
        xs = rt.scratch.get("ssm_x", (rt.max_tokens, H, P), f32)[:T]
        bs = rt.scratch.get("ssm_b", (rt.max_tokens, G, N), f32)[:T]
        cs = rt.scratch.get("ssm_c", (rt.max_tokens, G, N), f32)[:T]
        dts = rt.scratch.get("ssm_dt", (rt.max_tokens, H), f32)[:T]
        decay = rt.scratch.get("ssm_a", (rt.max_tokens, H), f32)[:T]
        S, conv = state["S"], state["conv"]
        ox, odt = self.inner, self.inner + self.conv_width
        kernels.ssm_prepare(proj, ox, odt, self.conv_w, self.conv_b, self.taps, conv, self.A_log, self.dt_bias,
                            step.entry_of_token, step.cu_q, step.state_slot, xs, bs, cs, dts, decay, H, P, G, N,
                            shift_single=True)
        # (requests that bring one token, which a step lists first, were moved on by the kernel above)
        kernels.conv_state_shift(proj[:, ox:ox + self.conv_width], self.taps, conv, step.cu_q, step.state_slot,
                                 step.n_entries - step.n_single, entry0=step.n_single)
        o = rt.scratch.get("ssm_o", (rt.max_tokens, H, P), f32)[:T]
        kernels.ssm_recurrence(cs, bs, xs, decay, dts, S, o, step.cu_q, step.state_slot, step.n_entries, G, H, N, P)
        y = rt.scratch.get("ssm_y", (rt.max_tokens, self.inner), rt.dtype)[:T]
        kernels.ssm_gate_norm(y, o, xs, proj, 0, self.skip, self.norm_w, H, P, self.parts, self.eps)
        out = rt.scratch.get(self.out_key, (rt.max_tokens, self.hidden), rt.dtype)[:T]
        return rt.linear(out, y, self.w_o)
