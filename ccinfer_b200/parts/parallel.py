"""A pair of mixers on the same rows, their results added with a constant factor each,

    out = left_scale * left(h) + right_scale * right(h).

What the pair keeps is what its halves keep: the cache of the one that has one (at most one of them may), and the
states of both (the step hands each half its own).
"""
from __future__ import annotations

from .. import kernels
from ..errors import Unsupported
from .base import Mixer


class ParallelMixers(Mixer):
    def __init__(self, hidden: int, left: Mixer, right: Mixer, left_scale: float, right_scale: float):
        if left.cache_need() is not None and right.cache_need() is not None:
            raise Unsupported("a pair of mixers on the same rows: at most one of them keeps a paged cache")
        self.hidden, self.left, self.right = int(hidden), left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        # each half leaves its result in a buffer of its own
        self.left.out_key, self.right.out_key = "mix_left_out", "mix_right_out"
        self.rt = None

    @property
    def graph_safe(self):
        return self.left.graph_safe and self.right.graph_safe

    @property
    def kernel_groups(self):
        return tuple(self.left.kernel_groups) + tuple(self.right.kernel_groups)

    @property
    def own_kv(self):
        return getattr(self.left, "own_kv", False) or getattr(self.right, "own_kv", False)

    def tensor_specs(self):
        return self.left.tensor_specs() + self.right.tensor_specs()

    def cache_need(self):
        return self.left.cache_need() or self.right.cache_need()

    @staticmethod
    def _needs(mixer, side):
        sn = mixer.state_need()
        if sn is None:
            return []
        sn = list(sn) if isinstance(sn, (list, tuple)) else [sn]
        import dataclasses
        return [dataclasses.replace(n, name=f"{side}.{n.name}") for n in sn]

    def state_need(self):
        needs = self._needs(self.left, "left") + self._needs(self.right, "right")
        return needs or None

    def bind(self, rt, fetch):
        self.rt = rt
        self.left.bind(rt, fetch)
        self.right.bind(rt, fetch)

    @staticmethod
    def _state_of(mixer, side, state):
        sn = mixer.state_need()
        if sn is None:
            return None
        if isinstance(sn, (list, tuple)):
            return {n.name: state[f"{side}.{n.name}"] for n in sn}
        return state[f"{side}.{sn.name}"]

    def forward(self, x, step, cache, state):
        rt = self.rt
        x = rt.rows(x)
        T = x.shape[0]
        lc = cache if self.left.cache_need() is not None else None
        rc = cache if self.right.cache_need() is not None else None
        a = self.left.forward(x, step, lc, self._state_of(self.left, "left", state))
        b = self.right.forward(x, step, rc, self._state_of(self.right, "right", state))
        out = rt.scratch.get(self.out_key, (rt.max_tokens, self.hidden), rt.dtype)[:T]
        kernels.scaled_sum(out, rt.rows(a), rt.rows(b), self.left_scale, self.right_scale)
        return out
