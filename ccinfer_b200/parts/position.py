"""Position encodings.

RotaryHalf: rotate-half rotation over the whole head,
inv_freq[i] = 1 / theta^(2i / head_dim), angle = float(pos) * inv_freq[i]
(7QiC/ccInfer: src/model/rope/rope_cache.cpp:31-45, src/kernel/pos/rope.cu:41-46).
The reference tabulates cos and sin for every position up to
max_position_embeddings on the host; here only the inverse frequencies are a
table and the kernel takes sine and cosine of the float angle, so no position
bound comes from a table.  The frequencies are evaluated as the reference
does, in 32-bit steps: exponent = float(2i) / float(head_dim), theta^exponent
rounded to float, 1.0f / that (a model trained with a 32-bit table sees the
frequencies it was trained with; evaluating in float64 and rounding once gives
another float for a third of the entries).  The power is taken in float64 and
rounded, i.e. correctly rounded, where the reference's powf is within an ulp.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import kernels
from .base import PositionEncoding


def rotary_inv_freq(rotary_dim: int, theta: float) -> np.ndarray:
    """float32 [rotary_dim / 2]: 1.0f / powf(theta, float(2i) / float(rotary_dim)), every step in 32 bits
    (src/model/rope/rope_cache.cpp:31-35)."""
    exponent = np.arange(0, rotary_dim, 2, dtype=np.float32) / np.float32(rotary_dim)
    power = np.power(np.float64(np.float32(theta)), exponent.astype(np.float64)).astype(np.float32)
    return (np.float32(1.0) / power).astype(np.float32)


class RotaryHalf(PositionEncoding):
    """Rotate-half rotation of the first ``rotary_dim`` coordinates of a head (default: all of them, as the
    reference: src/kernel/pos/rope.cu:37-46 pairs (i, i + head_dim / 2)).

    ``rotary_dim`` < head_dim: pairs (i, i + rotary_dim / 2), the other coordinates pass through.
    ``interleaved``: pairs (2i, 2i + 1) instead.  Both are a permutation of the head's coordinates into the
    kernels' layout plus a table with zeros for the pairs that do not turn (see PositionEncoding).
    """

    def __init__(self, head_dim: int, theta: float, rotary_dim: int = None, interleaved: bool = False,
                 linear_scaling: float = None, query_temperature=None, ramp_scaling: dict = None):
        """``linear_scaling`` s: every frequency is divided by s (positions are stretched by s); the table is
        then evaluated in float64 and rounded once.  ``query_temperature``: see ``QueryTemperature``.
        ``ramp_scaling`` {"factor", "original", "fast", "slow"}: only the slow pairs are stretched.  A pair that
        makes ``w`` full turns over ``original`` positions has the (fractional) number
        n(w) = rotary_dim * log(original / (w * 2 pi)) / (2 * log(theta)).  Pairs up to n(fast), rounded down and
        not below 0, keep their frequency; pairs from n(slow) on, rounded up and not above rotary_dim - 1, have it
        divided by ``factor``; between the two bounds the share b of the divided frequency grows linearly from 0 to
        1 (the bounds are kept at least 0.001 apart), freq = b * f / factor + (1 - b) * f.  Cosine and sine both
        carry the factor 1 + log(factor) / 10 (``amplitude``; the attention mixer puts it into the weights of its
        head norms)."""
        rotary_dim = int(head_dim if rotary_dim is None else rotary_dim)
        self.ramp_scaling = None
        if ramp_scaling is not None:
            if linear_scaling is not None:
                raise ValueError("linear_scaling or ramp_scaling, not both")
            self.ramp_scaling = {k: float(ramp_scaling[k]) for k in ("factor", "original", "fast", "slow")}
            if not (self.ramp_scaling["factor"] > 0 and self.ramp_scaling["original"] > 0
                    and self.ramp_scaling["fast"] > 0 and self.ramp_scaling["slow"] > 0):
                raise ValueError("ramp_scaling: factor, original, fast and slow must be > 0")
        if linear_scaling is not None and not (linear_scaling > 0):
            raise ValueError("linear_scaling must be > 0")
        self.linear_scaling = None if linear_scaling is None else float(linear_scaling)
        self._q_temp = query_temperature
        if head_dim % 2 or rotary_dim % 2 or not (0 < rotary_dim <= head_dim):
            raise ValueError(f"rotation of {rotary_dim} of {head_dim} coordinates: both even, 0 < rotary_dim <= head_dim")
        self.head_dim, self.theta, self.rotary_dim, self.interleaved = int(head_dim), float(theta), rotary_dim, interleaved
        self.inv_freq = None
        self.rt = None

    def bind(self, rt, fetch):
        self.rt = rt
        table = np.zeros(self.head_dim // 2, dtype=np.float32)
        if self.ramp_scaling is not None:
            table[:self.rotary_dim // 2] = self.ramp_frequencies().astype(np.float32)
        elif self.linear_scaling is None:
            table[:self.rotary_dim // 2] = rotary_inv_freq(self.rotary_dim, self.theta)
        else:
            i = np.arange(self.rotary_dim // 2, dtype=np.float64)
            table[:self.rotary_dim // 2] = (np.power(np.float64(self.theta), -2.0 * i / self.rotary_dim)
                                            / self.linear_scaling).astype(np.float32)
        self.inv_freq = torch.from_numpy(table).to(rt.device)

    def rotary_table(self):
        return self.inv_freq

    def ramp_frequencies(self) -> np.ndarray:
        """float64 [rotary_dim / 2]: the frequencies under ``ramp_scaling``."""
        import math
        sc, dims = self.ramp_scaling, self.rotary_dim
        f = np.power(np.float64(self.theta), -2.0 * np.arange(dims // 2, dtype=np.float64) / dims)

        def where(turns):
            return dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(self.theta))

        lo = max(math.floor(where(sc["fast"])), 0)
        hi = min(math.ceil(where(sc["slow"])), dims - 1)
        ramp = np.clip((np.arange(dims // 2, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / sc["factor"] * ramp + f * (1.0 - ramp)

    def amplitude(self):
        """None, or float32 [head_dim] in the kernels' layout: the factor on cosine and sine of each coordinate's
        pair (1 where a coordinate does not turn)."""
        if self.ramp_scaling is None:
            return None
        import math
        amp = 0.1 * math.log(self.ramp_scaling["factor"]) + 1.0
        half, rd = self.head_dim // 2, self.rotary_dim // 2
        v = np.ones(self.head_dim, dtype=np.float32)
        v[:rd] = amp
        v[half:half + rd] = amp
        return v

    def query_temperature(self):
        return self._q_temp

    def head_permutation(self):
        hd, rd, half = self.head_dim, self.rotary_dim, self.head_dim // 2
        if rd == hd and not self.interleaved:
            return None
        # the kernels' pair j is places (j, j + half): the rotated pairs first, then the rest in pairs of its own
        firsts = [2 * i for i in range(rd // 2)] if self.interleaved else list(range(rd // 2))
        seconds = [2 * i + 1 for i in range(rd // 2)] if self.interleaved else [i + rd // 2 for i in range(rd // 2)]
        rest = list(range(rd, hd))
        firsts += rest[:len(rest) // 2]
        seconds += rest[len(rest) // 2:]
        assert len(firsts) == len(seconds) == half
        return firsts + seconds

    def apply(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Rotates x [T, H, head_dim] on its own (the attention mixer fuses this with its cache write)."""
        T, H, hd = x.shape
        perm = self.head_permutation()
        if perm is not None:
            idx = torch.tensor(perm, device=x.device)
            x = x[..., idx].contiguous()
        out = torch.empty_like(x)
        kernels.qk_norm_rope_kv_write(x.view(T, H * hd), out, None, None, positions, None, self.inv_freq, None,
                                      None, 1.0, H, 0, hd, 1)
        if perm is not None:
            back = torch.empty_like(idx)
            back[idx] = torch.arange(hd, device=x.device)
            out = out[..., back].contiguous()
        return out


class NoPosition(PositionEncoding):
    """No position encoding at all."""

    def rotary_table(self):
        return None


class QueryTemperature(PositionEncoding):
    """No rotation; the position enters through the length of the query alone:
    q_p <- q_p * (1 + coef * ln(floor((p + 1) / every) + 1)), so that scores sharpen as the context grows
    in steps of ``every`` tokens.  Evaluated in float by the kernel that writes q."""

    def __init__(self, coef: float, every: int):
        if int(every) <= 0:
            raise ValueError("query temperature: 'every' must be a positive number of tokens")
        self.coef, self.every = float(coef), int(every)

    def rotary_table(self):
        return None

    def query_temperature(self):
        return (self.coef, self.every)
