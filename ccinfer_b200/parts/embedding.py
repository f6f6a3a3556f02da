"""Token embedding and output head.

  h0[t, :] = E[ids[t], :]                 (7QiC/ccInfer: src/kernel/elementwise/elementwise.cu:67-78)
  logits = x W_lm^T in float              (src/model/qwen3/qwen3_model.cpp:412-426)

The head runs on the rows whose logits are wanted, not on every token of the
step as the reference does.  A tied head names the embedding's tensor as its
weight and then shares its storage.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, Residual, StateNeed, TensorSpec


class TokenEmbedding(Part):
    def __init__(self, vocab: int, hidden: int, weight_name: str, scale: float = 1.0, pair: dict = None):
        """``scale``: the rows are multiplied by it (in float).  ``pair`` {"name", "buckets", "mul_prev", "mul_cur"}:
        a second table [buckets + 1, hidden]; the row added is hashed from the pair of tokens, (mul_prev * previous
        + mul_cur * current) % buckets, and at position 0 it is the table's last row.  The previous token is state of the request
        (``state_need``): a portion's first token finds it there."""
        self.vocab, self.hidden, self.weight_name = int(vocab), int(hidden), weight_name
        self.scale = float(scale)
        self.pair = dict(pair) if pair is not None else None
        if self.pair is not None:
            for k in ("buckets", "mul_prev", "mul_cur"):
                self.pair[k] = int(self.pair[k])
            if self.pair["buckets"] <= 0 or self.pair["mul_prev"] < 0 or self.pair["mul_cur"] < 0:
                raise ValueError("a pair table has buckets > 0 and multipliers >= 0")
        self.table = self.pair_table = None
        self.rt = None

    def tensor_specs(self):
        specs = [TensorSpec(self.weight_name, (self.vocab, self.hidden))]
        if self.pair is not None:
            specs.append(TensorSpec(self.pair["name"], (self.pair["buckets"] + 1, self.hidden)))
        return specs

    def state_need(self):
        """The previous token of each request, where a pair table is read."""
        return StateNeed((1,), torch.int32, "prev_token") if self.pair is not None else None

    def bind(self, rt, fetch):
        self.rt = rt
        self.table = fetch(self.weight_name)
        if self.pair is not None:
            self.pair_table = fetch(self.pair["name"])

    takes_first_norm = True

    def forward(self, step, first_norm=None, state=None) -> Residual:
        """``first_norm``: the norm that folds the stream first; where it can, its rows are written by the
        same kernel as the stream (``stream.ready``).  ``state``: the tensor of ``state_need``."""
        from .norm import StreamRows
        rt = self.rt
        h = rt.scratch.get("residual", (rt.max_tokens, self.hidden), torch.float32)[:step.n_tokens]
        pending = getattr(step, "pending_tokens", None)
        if self.pair is not None or self.scale != 1.0:
            rows = None
            if isinstance(first_norm, StreamRows) and rt.dtype != torch.float32:
                rows = first_norm.buffer(step.n_tokens)
            p = self.pair or {"buckets": 0, "mul_prev": 0, "mul_cur": 0}
            kernels.embed_pair(h, rows, self.table, self.pair_table, step.token_ids, step.positions,
                               step.entry_of_token, step.cu_q, step.state_slot,
                               state.view(-1) if state is not None else None, self.scale, p["buckets"], p["mul_prev"],
                               p["mul_cur"], step.n_entries, status=rt.status, pending=pending)
            stream = Residual(h)
            if rows is not None:
                stream.ready = (first_norm, rows)
            return stream
        y = None
        if first_norm is not None and hasattr(first_norm, "from_embedding"):
            y = first_norm.from_embedding(h, self.table, step.token_ids, pending)
        if y is None:
            kernels.embed_gather(h, self.table, step.token_ids, status=rt.status, pending=pending)
        stream = Residual(h)
        if y is not None:
            stream.ready = (first_norm, y)
        return stream


class TokenSideInput(Part):
    """A second, narrow embedding of the token that enters the stream after a layer, through a gate:

        e = table[token, offset : offset + dim];  g = gelu_tanh(Wgate h) * e;  y = Wproj g
        h += y / rms(y) * w_norm

    ``forward(h_rows, step)`` returns y (the caller sums it into the stream with its norm); the table is one
    tensor for all layers, each reading its own ``dim`` columns from ``offset``."""

    def __init__(self, vocab: int, hidden: int, dim: int, offset: int, table_width: int, eps: float, names: dict):
        """``names``: tensor names under the keys table, gate, proj, norm."""
        self.vocab, self.hidden, self.dim, self.offset = int(vocab), int(hidden), int(dim), int(offset)
        self.table_width, self.eps, self.names = int(table_width), float(eps), dict(names)
        self.w = None     # the norm's weight: the block's last sum applies it
        self.rt = None

    def tensor_specs(self):
        n = self.names
        return [TensorSpec(n["table"], (self.vocab, self.table_width)), TensorSpec(n["gate"], (self.dim, self.hidden)),
                TensorSpec(n["proj"], (self.hidden, self.dim)),
                TensorSpec(n["norm"], (self.hidden,), role="vector", init="one_plus_normal")]

    def bind(self, rt, fetch):
        self.rt = rt
        n = self.names
        self.table = fetch(n["table"])
        self.w_gate, self.w_proj = fetch(n["gate"]), fetch(n["proj"])
        self.w = fetch(n["norm"]).float().contiguous()

    def forward(self, h_rows: torch.Tensor, step) -> torch.Tensor:
        rt = self.rt
        T = h_rows.shape[0]
        g = rt.scratch.get("side_gate", (rt.max_tokens, self.dim), rt.dtype)[:T]
        rt.linear(g, h_rows, self.w_gate)
        kernels.gelu_gate_rows(g, self.table, self.offset, step.token_ids, status=rt.status,
                               pending=getattr(step, "pending_tokens", None))
        y = rt.scratch.get("side_out", (rt.max_tokens, self.hidden), rt.dtype)[:T]
        return rt.linear(y, g, self.w_proj)


class LoopInput(Part):
    """What a repeated pass over some layers starts from: h <- Win [h | h0] + step[t], h0 the embedding's rows,
    t the number of the pass (``Win`` [D, 2 D] with the stream's columns first, ``step`` [passes, D])."""

    def __init__(self, hidden: int, passes: int, names: dict):
        """``names``: tensor names under the keys in, step."""
        self.hidden, self.passes, self.names = int(hidden), int(passes), dict(names)
        self.rt = None

    needs_embedding = True

    def tensor_specs(self):
        D = self.hidden
        return [TensorSpec(self.names["in"], (D, 2 * D)), TensorSpec(self.names["step"], (self.passes, D), role="vector")]

    def bind(self, rt, fetch):
        self.rt = rt
        self.w_in = fetch(self.names["in"])
        self.steps = fetch(self.names["step"]).float().contiguous()

    def forward(self, stream: Residual, first_rows: torch.Tensor, number: int, step) -> None:
        rt = self.rt
        if stream.pending is not None:
            raise RuntimeError("the stream still has a sum pending where a pass begins")
        T, D = stream.h.shape
        both = rt.scratch.get("loop_rows", (rt.max_tokens, 2 * D), rt.dtype)[:T]
        kernels.concat_cast(both, stream.h, first_rows)
        rt.linear(stream.h, both, self.w_in)      # the product's rows are the float stream itself
        kernels.add_row(stream.h, self.steps[number])
        stream.ready = stream.unscaled = None


class OutputHead(Part):
    def __init__(self, hidden: int, vocab: int, weight_name: str):
        self.hidden, self.vocab, self.weight_name = int(hidden), int(vocab), weight_name
        self.w = None
        self.rt = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.vocab, self.hidden))]

    def bind(self, rt, fetch):
        self.rt = rt
        self.w = fetch(self.weight_name)

    def forward(self, x_rows: torch.Tensor) -> torch.Tensor:
        rt = self.rt
        R = x_rows.shape[0]
        if R <= rt.max_entries:  # the decode case: a fixed buffer, so that the step can be replayed
            logits = rt.scratch.get("logits", (rt.max_entries, self.vocab), torch.float32)[:R]
        else:
            logits = torch.empty((R, self.vocab), dtype=torch.float32, device=rt.device)
        rt.linear(logits, x_rows, self.w)
        return logits
