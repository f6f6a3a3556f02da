"""Mixture of experts: small feed-forward layers of which every token uses a few.

    z = Wr x (float);  s = softmax(z) over all experts;  choice score c = s + correction
    the experts form ``groups`` equal groups of neighbours; only experts of the ``keep`` groups with the largest
    best choice score can be chosen; the ``top`` largest c are chosen; their weights are their s, as they are
    m = sum_chosen s_e * Wdown_e act(Wup_e x)  +  Wdown_s act(Wup_s x)      (a shared expert for every token)

``activation`` "relu2": act(u) = relu(u)^2.  No biases.  ``activation`` "swiglu": every expert (the shared one
too) has a gate matrix beside its up matrix, act = silu(Wgate_e x) * (Wup_e x).  ``rule`` (``kernels.RouteRule``)
says how logits become scores and weights (sigmoid scores, a group's score as the sum of its two best, chosen
scores renormalised, a last factor); ``names["shared_gate"]``: the shared expert's result is multiplied by
sigmoid(w_sg . x), one number per token (the row rides along as one more row of the router's matrix).

Two forms, chosen by size (``sparse=`` forces one):

* dense, for experts so small that launches cost more than their arithmetic: every expert on every token as ONE
  product over all experts' first matrices (the shared expert's rows after them), an activation that multiplies
  each expert's columns by the token's weight for it (zero where it was not chosen), and ONE product with all
  second matrices side by side, which also adds the experts up;
* sparse: the (token, choice) pairs are sorted by expert and only the chosen experts run, as two grouped
  products over tiles of one expert's rows (``csrc/moe.cu``: mma.sync with operands straight from global memory
  for few rows an expert; ``csrc/moe_tcgen05.cu``: tcgen05 with TMA for many); the shared expert is two ordinary products; a last
  kernel adds each token's rows up in the order of its choices.  A decode step then reads the chosen experts'
  weights and no others.

Which form runs is settled when the weights are bound, and the weights are merged for that form.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import Unsupported
from .base import FeedForward, TensorSpec


class MixtureOfExperts(FeedForward):
    kernel_groups = ("moe",)
    # From this many weights of the routed experts on, the sparse form runs.  Measured on B200, bfloat16, 32 experts
    # of which 4 are chosen, the whole part in us, dense / sparse at 1, 8, 256, 2,048 tokens: 16.8 M weights
    # 22 / 26, 24 / 31, 37 / 51, 138 / 99; 67 M weights 47 / 33, 48 / 42, 75 / 78, 340 / 187.
    SPARSE_MIN_WEIGHTS = 1 << 25
    # (token, choice) pairs per expert from which the tcgen05 grouped product runs (402 M weights, 64 tokens, i.e.
    # 8 pairs an expert: 131 us against 222 us for tiles of 16 rows on mma.sync)
    TC_MIN_ROWS_PER_EXPERT = 8

    def __init__(self, hidden: int, experts: int, top: int, expert_ff: int, names: dict, groups: int = 1,
                 keep: int = 1, shared_ff: int = 0, activation: str = "relu2", sparse=None, rule=None):
        """``names``: "router", "correction" (optional), "up" and "down" (and "gate" with "swiglu") with ``{e}`` for
        the expert's number, "shared_up" / "shared_down" (/ "shared_gate_proj") with ``shared_ff`` > 0,
        "shared_gate" (optional)."""
        if activation not in ("relu2", "swiglu"):
            raise Unsupported(f"expert activation {activation!r}")
        self.glu = activation == "swiglu"
        self.rule = rule
        if experts % groups or not (0 < keep <= groups) or not (0 < top <= (experts // groups) * keep):
            raise Unsupported(f"{experts} experts in {groups} groups of which {keep} are kept cannot give {top}")
        self.hidden, self.E, self.top, self.F = int(hidden), int(experts), int(top), int(expert_ff)
        self.groups, self.keep, self.SF = int(groups), int(keep), int(shared_ff)
        self.names = dict(names)
        self.width = self.E * self.F + self.SF
        self.sparse = sparse
        self.rt = None

    def tensor_specs(self):
        n, D = self.names, self.hidden
        specs = [TensorSpec(n["router"], (self.E, D))]
        if n.get("correction"):
            specs.append(TensorSpec(n["correction"], (self.E,), role="vector"))
        for e in range(self.E):
            if self.glu:
                specs.append(TensorSpec(n["gate"].format(e=e), (self.F, D)))
            specs += [TensorSpec(n["up"].format(e=e), (self.F, D)), TensorSpec(n["down"].format(e=e), (D, self.F))]
        if self.SF:
            if self.glu:
                specs.append(TensorSpec(n["shared_gate_proj"], (self.SF, D)))
            specs += [TensorSpec(n["shared_up"], (self.SF, D)), TensorSpec(n["shared_down"], (D, self.SF))]
            if n.get("shared_gate"):
                specs.append(TensorSpec(n["shared_gate"], (1, D)))
        return specs

    def bind(self, rt, fetch):
        self.rt = rt
        n = self.names
        self.w_router = fetch(n["router"])
        self.has_shared_gate = bool(self.SF and n.get("shared_gate"))
        if self.has_shared_gate:   # its logit is column E of the router's product
            self.w_router = torch.cat([self.w_router, fetch(n["shared_gate"]).view(1, -1)], dim=0).contiguous()
        if self.glu:
            return self._bind_glu(rt, fetch)
        self.correction = fetch(n["correction"]).float().contiguous() if n.get("correction") else None
        ups = [fetch(n["up"].format(e=e)) for e in range(self.E)]
        downs = [fetch(n["down"].format(e=e)) for e in range(self.E)]
        # which form runs is settled here, by the sizes: the grouped products want 16-byte rows in bfloat16
        fits = rt.dtype == torch.float32 or (self.hidden % 8 == 0 and self.F % 8 == 0)
        big = 2 * self.E * self.F * self.hidden >= self.SPARSE_MIN_WEIGHTS
        self.use_sparse = fits and (big if self.sparse is None else bool(self.sparse))
        self.w_shared_up = self.w_shared_down = None
        if self.SF and self.use_sparse:      # the shared expert is two products of its own
            self.w_shared_up, self.w_shared_down = fetch(n["shared_up"]), fetch(n["shared_down"])
        elif self.SF:                        # its rows and columns come after the experts'
            ups.append(fetch(n["shared_up"]))
            downs.append(fetch(n["shared_down"]))
        self.w_up = torch.cat(ups, dim=0).contiguous()        # [E F (+ SF), D]
        self.w_down = torch.cat(downs, dim=1).contiguous()    # [D, E F (+ SF)]

    def _bind_glu(self, rt, fetch):
        """The gated form.  Dense: ONE matrix of all gate rows (the experts', then the shared expert's) followed by
        all up rows in the same order, and all second matrices side by side."""
        n = self.names
        self.correction = fetch(n["correction"]).float().contiguous() if n.get("correction") else None
        gates = [fetch(n["gate"].format(e=e)) for e in range(self.E)]
        ups = [fetch(n["up"].format(e=e)) for e in range(self.E)]
        downs = [fetch(n["down"].format(e=e)) for e in range(self.E)]
        fits = rt.dtype == torch.float32 or (self.hidden % 8 == 0 and self.F % 8 == 0)
        big = 3 * self.E * self.F * self.hidden >= self.SPARSE_MIN_WEIGHTS
        self.use_sparse = fits and (big if self.sparse is None else bool(self.sparse))
        self.w_shared_up = self.w_shared_down = None
        if self.use_sparse:
            # every expert's gate and up rows in turn (row 2 f its gate f, row 2 f + 1 its up f): a thread of the
            # grouped product holds both and the activation is its epilogue
            self.w_up = torch.stack([torch.stack([g, u], dim=1).reshape(2 * self.F, -1) for g, u in zip(gates, ups)]
                                    ).reshape(self.E * 2 * self.F, -1).contiguous()
            self.w_down = torch.cat(downs, dim=1).contiguous()
            if self.SF:
                self.w_shared_up = torch.cat([fetch(n["shared_gate_proj"]), fetch(n["shared_up"])], dim=0).contiguous()
                self.w_shared_down = fetch(n["shared_down"])
            return
        if self.SF:
            gates.append(fetch(n["shared_gate_proj"]))
            ups.append(fetch(n["shared_up"]))
            downs.append(fetch(n["shared_down"]))
        self.w_up = torch.cat(gates + ups, dim=0).contiguous()       # [2 (E F + SF), D]
        self.w_down = torch.cat(downs, dim=1).contiguous()           # [D, E F + SF]

    def _shared_gate(self, T):
        """The float column of the shared expert's gate logits in the router's product, or None."""
        if not self.has_shared_gate:
            return None
        rt = self.rt
        return rt.scratch.get("moe_logits", (rt.max_tokens, self.w_router.shape[0]), torch.float32)[:T, self.E]

    def route(self, x, T, sort_into=None):
        """idx int32 [T, top], wts float [T, top], dense float [T, E] for the rows of x.  ``sort_into`` (BM and the
        arrays of ``kernels.moe_sort``): the pairs are sorted by expert as well, in the same kernel where the step
        has few tokens (then there is no dense row)."""
        rt = self.rt
        logits = rt.scratch.get("moe_logits", (rt.max_tokens, self.w_router.shape[0]), torch.float32)[:T]
        rt.linear(logits, x, self.w_router)
        idx = rt.scratch.get("moe_idx", (rt.max_tokens, self.top), torch.int32)[:T]
        wts = rt.scratch.get("moe_wts", (rt.max_tokens, self.top), torch.float32)[:T]
        if sort_into is not None and T <= kernels.MOE_ROUTE_SORT_MAX_TOKENS:
            kernels.moe_route_sort(logits, self.correction, idx, wts, self.groups, self.keep, self.E, *sort_into,
                                   rule=self.rule)
            return idx, wts, None
        dense = rt.scratch.get("moe_dense", (rt.max_tokens, self.E), torch.float32)[:T]
        kernels.moe_route(logits, self.correction, idx, wts, dense, self.groups, self.keep, rule=self.rule, E=self.E)
        if sort_into is not None:
            kernels.moe_sort(idx, wts, self.E, *sort_into)
        return idx, wts, dense

    def _forward_sparse(self, x, T):
        rt = self.rt
        E, F, D, top = self.E, self.F, self.hidden, self.top
        i32, f32 = torch.int32, torch.float32
        pairs, max_pairs = T * top, rt.max_tokens * top
        # rows per tile: 16 (a decode step: the chosen experts' weights are streamed once per tile), or 128 on
        # tcgen05 once an expert gets some rows on average (bfloat16)
        tc = rt.dtype == torch.bfloat16 and pairs >= self.TC_MIN_ROWS_PER_EXPERT * E
        BM = kernels.MOE_TC_ROWS if tc else 16
        n_tiles = kernels.moe_max_tiles(pairs, E, BM)
        cap = kernels.moe_max_tiles(max_pairs, E, 16)
        # (layers of other sizes have buffers of their own: a buffer that only long steps use must not grow once
        # CUDA graphs hold the pool's addresses)
        src_row = rt.scratch.get(f"moe_src_row:{top}", (max_pairs,), i32)
        row_w = rt.scratch.get(f"moe_row_w:{top}", (max_pairs,), f32)
        pair_pos = rt.scratch.get(f"moe_pair_pos:{top}", (max_pairs,), i32)
        tiles = [rt.scratch.get(f"moe_tile{k}:{top}:{E}", (cap,), i32)[:n_tiles] for k in range(3)]
        idx, wts, _ = self.route(x, T, sort_into=(BM, src_row, row_w, pair_pos, *tiles))
        act = rt.scratch.get(f"moe_act_rows:{top}:{F}", (max_pairs, F), rt.dtype)[:pairs]
        rows = rt.scratch.get(f"moe_out_rows:{top}", (max_pairs, D), f32)[:pairs]
        # the first product's rows an expert and its mode: with gates, gate and up rows in turn and the gated
        # activation as the epilogue
        F1, first = (2 * F, 2) if self.glu else (F, 0)
        if tc:
            xs = rt.scratch.get(f"moe_x_sorted:{top}", (max_pairs, D), rt.dtype)[:pairs]
            kernels.moe_gather_rows(xs, x, src_row)
            kernels.moe_grouped_tc(act, xs, self.w_up, row_w, *tiles, F1, D, F1, first, status=rt.status)
            kernels.moe_grouped_tc(rows, act, self.w_down, row_w, *tiles, D, F, F, 1, status=rt.status)
        else:
            kernels.moe_grouped(act, x, src_row, self.w_up, F1 * self.w_up.stride(0), row_w, *tiles, F1, D, BM, first)
            kernels.moe_grouped(rows, act, None, self.w_down, F, row_w, *tiles, D, F, BM, 1)
        shared = None
        if self.SF and self.glu:
            sa = rt.scratch.get(f"moe_shared_act:{self.SF}", (rt.max_tokens, self.SF), rt.dtype)[:T]
            gu = rt.scratch.get(f"moe_shared_gate_up:{self.SF}", (rt.max_tokens, 2 * self.SF), rt.dtype)[:T]
            rt.linear(gu, x, self.w_shared_up)
            kernels.moe_dense_glu_act(sa, gu, None, 0, 1, self.SF, self._shared_gate(T))
            shared = rt.scratch.get("moe_shared_out", (rt.max_tokens, D), rt.dtype)[:T]
            rt.linear(shared, sa, self.w_shared_down)
        elif self.SF:
            sa = rt.scratch.get(f"moe_shared_act:{self.SF}", (rt.max_tokens, self.SF), rt.dtype)[:T]
            rt.linear(sa, x, self.w_shared_up)
            kernels.moe_dense_act(sa, wts, 0, 1, self.SF)
            shared = rt.scratch.get("moe_shared_out", (rt.max_tokens, D), rt.dtype)[:T]
            rt.linear(shared, sa, self.w_shared_down)
        out = rt.scratch.get("ffn_out", (rt.max_tokens, D), rt.dtype)[:T]
        kernels.moe_combine(out, rows, pair_pos, shared, top)
        return out

    def forward(self, x, step):
        rt = self.rt
        x = rt.rows(x)
        T = x.shape[0]
        if self.use_sparse:
            return self._forward_sparse(x, T)
        _, _, dense = self.route(x, T)
        act = rt.scratch.get("moe_act", (rt.max_tokens, self.width), rt.dtype)[:T]
        if self.glu:
            gu = rt.scratch.get("moe_gate_up", (rt.max_tokens, 2 * self.width), rt.dtype)[:T]
            rt.linear(gu, x, self.w_up)
            kernels.moe_dense_glu_act(act, gu, dense, self.E, self.F, self.SF, self._shared_gate(T))
        else:
            rt.linear(act, x, self.w_up)
            kernels.moe_dense_act(act, dense, self.E, self.F, self.SF)
        out = rt.scratch.get("ffn_out", (rt.max_tokens, self.hidden), rt.dtype)[:T]
        return rt.linear(out, act, self.w_down)
