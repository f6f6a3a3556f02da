"""Arrangements of parts in a block.

PostNormBlock: h += post1(Mixer(h)); h += post2(FeedForward(h)): a norm on each sublayer's output only.

PreNormBlock: a = Mixer(norm1(h)); h += a; m = FeedForward(norm2(h)); h += m
(7QiC/ccInfer: src/model/qwen3/qwen3_model.cpp:141-396).  Each sum is folded
into the norm that follows it, the last one into the model's final norm.
The last product of the mixer and of the feed-forward is offered a
``ResidualSink``: with few rows it adds its result to the stream itself and the
norm after it needs no kernel (``parts.base.UnscaledRows``).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import Block, FeedForward, Mixer, Norm, Residual, ResidualSink


def _groups_of(parts):
    return tuple(dict.fromkeys(g for p in parts for g in getattr(p, "kernel_groups", ())))


class PreNormBlock(Block):
    """h += Mixer(norm1(h)); h += FeedForward(norm2(h)); optionally, last, h += side(h, token).

    The feed-forward (with norm2) may be absent.  ``side`` (``parts.embedding.TokenSideInput``): the block's last
    sum also writes the stream's rows in the compute type for the side input's gate, and the side input's own sum
    (with its RMS norm) writes the first norm of the block that follows (``stream.ready``)."""

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm] = None, ffn: Optional[FeedForward] = None,
                 side=None):
        if (ffn is None) != (norm2 is None):
            raise ValueError("a feed-forward comes with its norm, or neither is given")
        self.norm1, self.mixer, self.norm2, self.ffn, self.side = norm1, mixer, norm2, ffn, side
        self.rt = None

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn, self.side) if p is not None]

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self._parts())

    @property
    def kernel_groups(self):
        return _groups_of(self._parts())

    def tensor_specs(self):
        return [s for p in self._parts() for s in p.tensor_specs()]

    def bind(self, rt, fetch):
        self.rt = rt
        for p in self._parts():
            p.bind(rt, fetch)
        self._ones = None
        if self.side is not None:   # the plain sum as the kernel that sums with a factor per channel
            self._ones = torch.ones(self.side.hidden, dtype=torch.float32, device=rt.device)

    @property
    def first_norm(self):
        return self.norm1

    def forward(self, stream: Residual, step, cache, state) -> None:
        after = stream.next_norm                     # the norm that the block after this one starts with
        if self.side is not None:
            after = None                             # (the side input's sum writes that norm's rows itself)
        stream.takes_unscaled = self.mixer.takes_unscaled
        x = self.norm1.fold(stream)
        nxt = self.norm2 if self.ffn is not None else after
        step.residual_sink = ResidualSink(stream, nxt) if nxt is not None else None
        stream.pending = self.mixer.forward(x, step, cache, state)
        if self.ffn is not None:
            stream.takes_unscaled = self.ffn.takes_unscaled
            x = self.norm2.fold(stream)
            step.residual_sink = ResidualSink(stream, after) if after is not None else None
            stream.pending = self.ffn.forward(x, step)
        step.residual_sink = None
        stream.takes_unscaled = False
        if self.side is not None:
            self._side(stream, step)

    def _side(self, stream: Residual, step) -> None:
        """h += pending, then h += side(h, token) with the side input's norm, in two kernels that also write what
        reads the stream next (the stream's rows for the side input's gate; the next block's first norm)."""
        rt = self.rt
        T, D = stream.h.shape
        after = stream.next_norm
        rows = rt.scratch.get("stream_rows", (rt.max_tokens, D), rt.dtype)[:T]
        delta, stream.pending = stream.pending, None
        if delta is None:
            raise RuntimeError("the block's last part left nothing to add where a side input follows")
        stream.unscaled = stream.ready = None
        kernels.scaled_residual(stream.h, rt.rows(delta), self._ones, y=rows)
        y = self.side.forward(rows, step)
        usable = after is not None and hasattr(after, "w") and hasattr(after, "eps")
        x = rt.scratch.get(after.scratch_key, (rt.max_tokens, D), rt.dtype)[:T] if usable else None
        kernels.postnorm_residual(stream.h, rt.rows(y), self.side.w, 1.0, self.side.eps, y=x,
                                  w_next=after.w if usable else None, eps_next=after.eps if usable else 0.0)
        stream.ready = (after, x) if usable else None


class SandwichNormBlock(Block):
    """A norm before AND after each sublayer, the normed output scaled by a constant before the sum:

        h += mult * post1(Mixer(norm1(h)));   h += mult * post2(FeedForward(norm2(h)))

    The feed-forward (with norm2 and post2) may be absent.  All four are RMS norms with the same eps.  The
    sum, the norm of the sublayer's output and the norm that reads the stream next are one kernel
    (``kernels.postnorm_residual``): it also takes the rows that a repeated pass adds to the stream
    (``Residual.next_add``) and leaves the next block's first norm as ``stream.ready``."""

    def __init__(self, norm1, mixer: Mixer, post1, norm2=None, ffn: Optional[FeedForward] = None, post2=None,
                 mult: float = 1.0):
        if (ffn is None) != (norm2 is None) or (ffn is None) != (post2 is None):
            raise ValueError("a feed-forward comes with its two norms, or none of the three is given")
        self.norm1, self.mixer, self.post1, self.norm2, self.ffn, self.post2 = norm1, mixer, post1, norm2, ffn, post2
        self.mult = float(mult)
        self.rt = None

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.post1, self.norm2, self.ffn, self.post2) if p is not None]

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self._parts())

    @property
    def kernel_groups(self):
        return _groups_of(self._parts())

    def tensor_specs(self):
        return [s for p in self._parts() for s in p.tensor_specs()]

    def bind(self, rt, fetch):
        self.rt = rt
        for p in self._parts():
            p.bind(rt, fetch)

    @property
    def first_norm(self):
        return self.norm1

    def _sum(self, stream: Residual, delta, post, nxt, last: bool):
        """h += mult * post(delta) (+ the rows a repeated pass adds, after the block's last sum); with
        ``nxt`` its rows are returned."""
        rt = self.rt
        add = None
        if last and stream.next_add is not None:
            add, stream.next_add = stream.next_add, None
        y = None
        usable = nxt is not None and hasattr(nxt, "w") and hasattr(nxt, "eps")
        if usable:
            y = rt.scratch.get(nxt.scratch_key, (rt.max_tokens, nxt.dim), rt.dtype)[:stream.h.shape[0]]
        kernels.postnorm_residual(stream.h, rt.rows(delta), post.w, self.mult, post.eps, add=add,
                                  y=y, w_next=nxt.w if usable else None, eps_next=nxt.eps if usable else 0.0)
        return y

    def forward(self, stream: Residual, step, cache, state) -> None:
        after = stream.next_norm
        stream.takes_unscaled = False
        x = self.norm1.fold(stream)
        step.residual_sink = None
        a = self.mixer.forward(x, step, cache, state)
        x = self._sum(stream, a, self.post1, self.norm2 if self.ffn is not None else after, self.ffn is None)
        if self.ffn is not None:
            m = self.ffn.forward(x, step)
            x = self._sum(stream, m, self.post2, after, True)
        stream.ready = (after, x) if (after is not None and x is not None) else None


class LayerScaleBlock(Block):
    """Pre-norm with a factor per channel on each sublayer's output, and optionally a token side input last:

        h += ls1 * Mixer(norm1(h));   h += ls2 * FeedForward(norm2(h));   h += side(h, token)

    The feed-forward (with norm2 and ls2) may be absent.  Each sum is one kernel that also writes what reads the
    stream next: the next norm's rows, or the stream's own rows in the compute type for the side input's gate.
    The side input's sum (with its RMS norm) writes the first norm of the block that follows (``stream.ready``).
    ``ls_names``: the tensors of ls1 and ls2."""

    def __init__(self, dim: int, norm1, mixer: Mixer, ls_names, norm2=None, ffn: Optional[FeedForward] = None,
                 side=None):
        if (ffn is None) != (norm2 is None):
            raise ValueError("a feed-forward comes with its norm, or neither is given")
        self.dim, self.norm1, self.mixer, self.norm2, self.ffn, self.side = int(dim), norm1, mixer, norm2, ffn, side
        self.ls_names = tuple(ls_names)
        self.rt = None

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn, self.side) if p is not None]

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self._parts())

    @property
    def kernel_groups(self):
        return _groups_of(self._parts())

    def tensor_specs(self):
        from .base import TensorSpec
        specs = [s for p in self._parts() for s in p.tensor_specs()]
        n = 2 if self.ffn is not None else 1
        return specs + [TensorSpec(name, (self.dim,), role="vector", init="one_plus_normal") for name in self.ls_names[:n]]

    def bind(self, rt, fetch):
        self.rt = rt
        for p in self._parts():
            p.bind(rt, fetch)
        self.ls1 = fetch(self.ls_names[0]).float().contiguous()
        self.ls2 = fetch(self.ls_names[1]).float().contiguous() if self.ffn is not None else None

    @property
    def first_norm(self):
        return self.norm1

    def _rows_buffer(self, key, T):
        rt = self.rt
        return rt.scratch.get(key, (rt.max_tokens, self.dim), rt.dtype)[:T]

    def _sum(self, stream, delta, ls, nxt, last: bool):
        """h += ls * delta; returns the rows of what reads the stream next: ``nxt``'s (a norm with a weight and
        an eps), the stream's own rows in the compute type before a side input, or None."""
        rt = self.rt
        T = stream.h.shape[0]
        delta = rt.rows(delta)
        if last and self.side is not None:
            rows = self._rows_buffer("stream_rows", T)
            kernels.scaled_residual(stream.h, delta, ls, y=rows)
            return rows
        if nxt is not None and hasattr(nxt, "w") and hasattr(nxt, "eps"):
            y = self._rows_buffer(nxt.scratch_key, T)
            kernels.scaled_residual(stream.h, delta, ls, y=y, w_next=nxt.w, eps_next=nxt.eps)
            return y
        kernels.scaled_residual(stream.h, delta, ls)
        return None

    def forward(self, stream: Residual, step, cache, state) -> None:
        rt = self.rt
        after = stream.next_norm
        stream.takes_unscaled = False
        x = self.norm1.fold(stream)
        step.residual_sink = None
        a = self.mixer.forward(x, step, cache, state)
        x = self._sum(stream, a, self.ls1, self.norm2 if self.ffn is not None else after, self.ffn is None)
        if self.ffn is not None:
            m = self.ffn.forward(x, step)
            x = self._sum(stream, m, self.ls2, after, True)
        if self.side is not None:
            y = self.side.forward(x, step)
            usable = after is not None and hasattr(after, "w") and hasattr(after, "eps")
            x = self._rows_buffer(after.scratch_key, stream.h.shape[0]) if usable else None
            kernels.postnorm_residual(stream.h, rt.rows(y), self.side.w, 1.0, self.side.eps, y=x,
                                      w_next=after.w if usable else None, eps_next=after.eps if usable else 0.0)
        stream.ready = (after, x) if (after is not None and x is not None) else None


class PostNormBlock(Block):
    """A norm on each sublayer's OUTPUT only; the sublayers read the stream itself:

        h += post1(Mixer(h));   h += post2(FeedForward(h))

    The feed-forward (with post2) may be absent.  Each sum is one kernel (``kernels.postnorm_residual``) that norms
    the sublayer's output, adds it and writes what reads the stream next: the stream's own rows in the compute type
    (for this block's feed-forward, or for a block after it that starts the same way: ``stream.ready``), or the
    rows of the norm that the block after it starts with.  In the 32-bit path the sublayers get the stream's
    tensor itself."""

    def __init__(self, dim: int, mixer: Mixer, post1, ffn: Optional[FeedForward] = None, post2=None):
        from .norm import StreamRows
        if (ffn is None) != (post2 is None):
            raise ValueError("a feed-forward comes with its norm, or neither is given")
        self.dim, self.mixer, self.post1, self.ffn, self.post2 = int(dim), mixer, post1, ffn, post2
        self.reads = StreamRows(dim)
        self.rt = None

    def _parts(self):
        return [p for p in (self.reads, self.mixer, self.post1, self.ffn, self.post2) if p is not None]

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self._parts())

    @property
    def kernel_groups(self):
        return _groups_of(self._parts())

    def tensor_specs(self):
        return [s for p in self._parts() for s in p.tensor_specs()]

    def bind(self, rt, fetch):
        self.rt = rt
        for p in self._parts():
            p.bind(rt, fetch)

    @property
    def first_norm(self):
        return self.reads

    def _sum(self, stream: Residual, delta, post, nxt):
        """h += post(delta); returns (what ``nxt`` reads, or None): ``nxt`` is a ``StreamRows`` (the stream's own
        rows) or a norm with a weight and an eps."""
        from .norm import StreamRows
        rt = self.rt
        T = stream.h.shape[0]
        y = w_next = None
        eps_next = 0.0
        if isinstance(nxt, StreamRows):
            y = None if rt.dtype == torch.float32 else nxt.buffer(T)
        elif nxt is not None and hasattr(nxt, "w") and hasattr(nxt, "eps"):
            y = rt.scratch.get(nxt.scratch_key, (rt.max_tokens, nxt.dim), rt.dtype)[:T]
            w_next, eps_next = nxt.w, nxt.eps
        kernels.postnorm_residual(stream.h, rt.rows(delta), post.w, 1.0, post.eps, y=y, w_next=w_next,
                                  eps_next=eps_next)
        if isinstance(nxt, StreamRows):
            return stream.h if y is None else y
        return y

    def forward(self, stream: Residual, step, cache, state) -> None:
        after = stream.next_norm
        stream.takes_unscaled = False
        x = self.reads.fold(stream)
        step.residual_sink = None
        a = self.mixer.forward(x, step, cache, state)
        x = self._sum(stream, a, self.post1, self.reads if self.ffn is not None else after)
        if self.ffn is not None:
            m = self.ffn.forward(x, step)
            x = self._sum(stream, m, self.post2, after)
        if stream.next_add is not None:
            x = None   # the engine adds the embedding's rows next: what was written ahead no longer holds
        stream.ready = (after, x) if (after is not None and x is not None) else None
