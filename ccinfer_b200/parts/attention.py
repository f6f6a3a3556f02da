"""Grouped-query attention over a paged cache.

  [q|k|v] = x W_qkv^T (no bias); optional per-head RMSNorm of q and k over the
  head axis, before the rotation; rotate-half position encoding of q and k; k
  (rotated) and v go to the cache; q head h reads kv head h / (nq / nkv);
  s = q.k / sqrt(hd), causal (optionally windowed) softmax, o = P v; a = o W_o^T
  (7QiC/ccInfer: src/model/qwen3/qwen3_model.cpp:158-298).

The three projections are one merged matrix (rows q, then k, then v), as the
reference merges them at load (src/model/qwen3/qwen3_weights.cpp:16-43).  A
layer that reads another layer's cache (``own_kv=False``) has only the q and
o projections (and must use the position encoding of the layer whose keys it
reads).  Head sizes are multiples of 16 up to 256: others are refused (the
reference's decode kernel takes any head size up to 128,
src/kernel/attention/decode_attn.cu:521-569).

Beyond the reference: biases of the three projections (names q_bias, k_bias,
v_bias; added by the kernel that rotates q and k and writes the cache), a
value size that differs from the query/key size (``value_dim``), a score scale
of the model's choosing, and a query temperature stated by the position
encoding (both also inside the fused decode attention).  The attention kernels know one head size; with ``value_dim`` given,
the heads of q, k and v are laid out in the smallest size the kernels take that
holds both (a multiple of 16), the added coordinates being zero rows of the
projections and zero columns of the output projection: zeros in q and k add
nothing to a score, zeros in v give zeros that the output projection ignores.
Per-head norms of q and k over heads laid out in a larger size keep their own
divisor: the mean over ``head_dim`` coordinates is the mean over the laid-out
ones times a constant, which goes into the bound weights and the eps.

Further options, each with its constants as arguments: a short causal
convolution over time on every channel of q, k and v directly after the
projection (``conv_taps``; the last taps - 1 projected rows of a request are its
state); a chunked mask (``chunk``: a query sees the keys of its own run of that
many positions, counted from the sequence's start); a learned sink per head in
the softmax denominator (name ``sink``); values mixed with those of the first
such layer, v <- (1 - lambda) v + lambda v_first, before they are cached
(``value_mix``); and a gate per head on the result, sigmoid(w_g . x), read from
the same input as the projections (name ``gate``; its rows ride along in the
merged projection); heads that talk to each other before the softmax (names
``talk`` [heads, heads] and optionally ``temp`` [heads]): head h's score is
sum_g talk[h, g] * temp[g] * scale * (q_g . k), which one kernel computes for
all heads of a query together (``csrc/attention_talking.cu``); a position
encoding with an amplitude on its rotation (``PositionEncoding.amplitude``).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import kernels
from ..errors import Unsupported
from .base import CacheNeed, Mixer, PositionEncoding, StateNeed, TensorSpec


class GroupedQueryAttention(Mixer):
    takes_unscaled = True

    @property
    def kernel_groups(self):
        groups = ["talking"] if self.talking else ["attention"]
        if self.taps or self.value_mix is not None:
            groups.append("recurrent")   # (the short convolutions live there)
        return tuple(groups)

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PositionEncoding, names: dict, qk_norm_eps: Optional[float] = None,
                 window: Optional[int] = None, own_kv: bool = True, scale: Optional[float] = None,
                 value_dim: Optional[int] = None, float_weights: bool = False, chunk: Optional[int] = None,
                 conv_taps: int = 0, value_mix: Optional[tuple] = None):
        """``names``: tensor names under the keys q, k, v, o and (with qk_norm_eps) q_norm, k_norm; with
        q_bias, k_bias, v_bias the projections have biases; ``sink`` [heads]; ``gate`` [heads, hidden]; with
        ``conv_taps`` > 0 q_conv, k_conv, v_conv ([channels, taps]).  ``value_mix``: ("first", key) — this
        layer's values are kept for the step under ``key``; ("mix", key) — its values are mixed with those,
        lambda the scalar tensor named ``vmix``.  ``value_dim``: size of a value head where it is
        not ``head_dim``; the position encoding is then built for ``kernel_head_dim(head_dim, value_dim)``.
        ``float_weights``: the softmax weights stay float up to their product with the values (every row
        goes to the split kernel; the tensor-core kernels round them to bfloat16 for that product)."""
        if num_heads % num_kv_heads:
            raise Unsupported(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        self.qk_dim = int(head_dim)
        self.v_dim = int(head_dim if value_dim is None else value_dim)
        if value_dim is not None:
            head_dim = self.kernel_head_dim(head_dim, value_dim)
        if head_dim % 16 or head_dim > 256:
            raise Unsupported(f"head size {head_dim}: the attention kernels take multiples of 16 up to 256")
        if window is not None and window <= 0:
            raise Unsupported("a window must be > 0")
        self.hidden, self.nq, self.nkv, self.hd = int(hidden), int(num_heads), int(num_kv_heads), int(head_dim)
        self.position, self.names = position, dict(names)
        self.qk_norm_eps, self.window, self.own_kv = qk_norm_eps, window, own_kv
        self.has_bias = "q_bias" in self.names
        self.chunk = int(chunk) if chunk else 0
        self.taps = int(conv_taps) if conv_taps else 0
        if self.chunk < 0 or self.taps < 0 or self.taps > 16:
            raise Unsupported(f"chunk {chunk}, {conv_taps} taps: a chunk is > 0, a convolution has 1 to 16 taps")
        if value_mix is not None and (len(value_mix) != 2 or value_mix[0] not in ("first", "mix")):
            raise Unsupported(f"value_mix {value_mix!r}: ('first', key) or ('mix', key)")
        self.value_mix = tuple(value_mix) if value_mix is not None else None
        if (self.taps or self.value_mix or "gate" in self.names) and not own_kv:
            raise Unsupported("a layer that reads another layer's keys has no convolution, value mixing or gate")
        if (self.taps or self.value_mix) and self.has_bias:
            raise Unsupported("biases together with a convolution or value mixing")
        # attention beyond keys and values (every attention kernel takes them)
        self.extras = bool(self.chunk or "sink" in self.names or "gate" in self.names)
        self.talking = "talk" in self.names
        if "temp" in self.names and not self.talking:
            raise Unsupported("a temperature per head comes with the heads' mixing matrix ('talk')")
        if self.talking and self.chunk:
            raise Unsupported("heads that talk to each other together with a chunked mask")
        self.mix = None
        self.float_weights = bool(float_weights)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.qk_dim)
        self.q_width, self.kv_width = self.nq * self.hd, self.nkv * self.hd
        self.conv_width = self.q_width + 2 * self.kv_width      # the columns a convolution runs over: q | k | v
        self.gate_off = self.conv_width                         # the gate's columns come after them
        self.in_width = self.conv_width + (-(-self.nq // 8) * 8 if "gate" in self.names else 0)
        self.bias = self.sink = self.conv_w = self.vmix = None
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None
        self.rt = None

    @staticmethod
    def kernel_head_dim(head_dim: int, value_dim: int) -> int:
        """The head size the kernels run with for these query/key and value sizes."""
        return -(-max(int(head_dim), int(value_dim)) // 16) * 16

    # -- what it wants ---------------------------------------------------------
    def tensor_specs(self):
        n, D = self.names, self.hidden
        specs = [TensorSpec(n["q"], (self.nq * self.qk_dim, D)), TensorSpec(n["o"], (D, self.nq * self.v_dim))]
        if self.own_kv:
            specs += [TensorSpec(n["k"], (self.nkv * self.qk_dim, D)), TensorSpec(n["v"], (self.nkv * self.v_dim, D))]
        if self.has_bias:
            specs.append(TensorSpec(n["q_bias"], (self.nq * self.qk_dim,), role="vector"))
            if self.own_kv:
                specs += [TensorSpec(n["k_bias"], (self.nkv * self.qk_dim,), role="vector"),
                          TensorSpec(n["v_bias"], (self.nkv * self.v_dim,), role="vector")]
        if self.qk_norm_eps is not None:
            specs.append(TensorSpec(n["q_norm"], (self.qk_dim,), role="vector", init="one_plus_normal"))
            if self.own_kv:
                specs.append(TensorSpec(n["k_norm"], (self.qk_dim,), role="vector", init="one_plus_normal"))
        if self.taps:
            specs += [TensorSpec(n["q_conv"], (self.nq * self.qk_dim, self.taps), role="vector"),
                      TensorSpec(n["k_conv"], (self.nkv * self.qk_dim, self.taps), role="vector"),
                      TensorSpec(n["v_conv"], (self.nkv * self.v_dim, self.taps), role="vector")]
        if "sink" in n:
            specs.append(TensorSpec(n["sink"], (self.nq,), role="vector"))
        if "gate" in n:
            specs.append(TensorSpec(n["gate"], (self.nq, D)))
        if self.talking:
            specs.append(TensorSpec(n["talk"], (self.nq, self.nq), role="vector"))
            if "temp" in n:
                specs.append(TensorSpec(n["temp"], (self.nq,), role="vector", init="one_plus_normal"))
        if "vmix" in n:   # (a layer whose values are the first ones may carry the tensor without using it)
            specs.append(TensorSpec(n["vmix"], (), role="vector"))
        return specs

    def cache_need(self):
        return CacheNeed.keys_and_values(self.nkv, self.hd, self.window, chunk=self.chunk or None)

    def state_need(self):
        if self.taps > 1:   # the last taps - 1 rows of the q | k | v projection
            return StateNeed((self.taps - 1, self.conv_width), dtype=None, name="conv")
        return None

    def bind(self, rt, fetch):
        self.rt = rt
        n = self.names
        self.position.bind(rt, fetch)
        if self.position.score_bias() is not None:
            raise Unsupported("a position encoding that adds to the scores: the attention kernels take rotations "
                              "of q and k only")
        table = self.position.rotary_table()
        if table is not None and (table.dtype != torch.float32 or table.numel() != self.hd // 2):
            raise Unsupported(f"a rotary table of {self.hd // 2} float frequencies is wanted for head size "
                              f"{self.hd}, the position encoding gives {tuple(table.shape)} {table.dtype}")
        # the encoding's own pairing of coordinates, brought into the kernels' layout (pairs (j, j + hd / 2))
        # by permuting the rows of the query and key projections and the head norms' weights alike
        perm = self.position.head_permutation()
        if perm is not None:
            if sorted(perm) != list(range(self.hd)):
                raise Unsupported(f"head_permutation() must name each of the {self.hd} coordinates once")
            idx = torch.tensor(perm, device=rt.device)

            def heads(w, n_heads):
                return w.view(n_heads, self.hd, -1)[:, idx, :].reshape(n_heads * self.hd, -1)
        else:
            idx = None

            def heads(w, n_heads):
                return w
        hd = self.hd

        def laid_out(w, n_heads, d):
            """[n_heads * d, ...] -> [n_heads * hd, ...]: each head's rows followed by zero rows up to hd."""
            if d == hd:
                return w
            w = w.view(n_heads, d, -1)
            out = torch.zeros((n_heads, hd, w.shape[2]), dtype=w.dtype, device=w.device)
            out[:, :d] = w
            return out.view(n_heads * hd, -1)

        def qk(name, n_heads):
            return heads(laid_out(fetch(n[name]), n_heads, self.qk_dim), n_heads)

        if self.own_kv:
            mats = [qk("q", self.nq), qk("k", self.nkv), laid_out(fetch(n["v"]), self.nkv, self.v_dim)]
            if "gate" in n:
                gate = torch.zeros((self.in_width - self.conv_width, self.hidden), dtype=mats[0].dtype, device=rt.device)
                gate[:self.nq] = fetch(n["gate"])
                mats.append(gate)
            self.w_qkv = torch.cat(mats, dim=0).contiguous()
        else:
            self.w_qkv = qk("q", self.nq).contiguous()
        if self.has_bias:
            parts = [qk("q_bias", self.nq)]
            if self.own_kv:
                parts += [qk("k_bias", self.nkv), laid_out(fetch(n["v_bias"]), self.nkv, self.v_dim)]
            self.bias = torch.cat([p.reshape(-1) for p in parts]).float().contiguous()
        w_o = fetch(n["o"])
        if self.v_dim != hd:   # zero columns where the heads of o carry the added coordinates
            w_o = laid_out(w_o.t().contiguous(), self.nq, self.v_dim).t().contiguous()
        self.w_o = w_o
        self.norm_eps = self.qk_norm_eps
        if self.qk_norm_eps is not None:
            def norm_w(name):
                w = fetch(n[name]).float()
                if self.qk_dim != hd:
                    # the kernels divide the sum of squares by hd: 1 / sqrt(ss / d + eps) =
                    # sqrt(d / hd) / sqrt(ss / hd + eps d / hd), and the added coordinates are zero
                    w = torch.cat([w * math.sqrt(self.qk_dim / hd), torch.zeros(hd - self.qk_dim, device=w.device)])
                return (w[idx] if idx is not None else w).contiguous()
            self.q_norm_w = norm_w("q_norm")
            self.k_norm_w = norm_w("k_norm") if self.own_kv else None
            self.norm_eps = self.qk_norm_eps * self.qk_dim / hd
        amp = self.position.amplitude()
        if amp is not None:
            # a factor on cosine and sine is a factor on the rotated coordinate: it rides on the norms' weights
            if self.qk_norm_eps is None:
                raise Unsupported("a rotation with an amplitude needs the head norms whose weights carry it")
            amp = torch.from_numpy(amp).to(rt.device)
            self.q_norm_w = (self.q_norm_w * amp).contiguous()
            if self.k_norm_w is not None:
                self.k_norm_w = (self.k_norm_w * amp).contiguous()
        if self.talking:
            if not kernels.attention_talking_fits(self.nq, self.nkv, hd):
                raise Unsupported(f"{self.nq} heads of {hd} that talk to each other: the kernel's shared memory "
                                  f"holds every head's query and result rows of a token")
            mix = fetch(n["talk"]).double()
            if "temp" in n:
                mix = mix * fetch(n["temp"]).double()[None, :]
            self.mix = (mix * self.scale).float().contiguous()
        if self.taps:
            # tap-major for the kernel: [taps, q | k | v channels]
            self.conv_w = torch.cat([qk("q_conv", self.nq), qk("k_conv", self.nkv),
                                     laid_out(fetch(n["v_conv"]), self.nkv, self.v_dim)], dim=0).float().t().contiguous()
        if "sink" in n:
            self.sink = fetch(n["sink"]).float().contiguous()
        if self.value_mix is not None and self.value_mix[0] == "mix":
            self.vmix = fetch(n["vmix"]).float().reshape(1).contiguous()

    def _attend(self, q, o, cache, step, T, gate=None):
        """Attention of every token row of the step over its request's pages.

        A step lists its single-token requests first.  On the tensor-core path (bfloat16, head size 64 or
        128) those rows go to the decode kernel (key range split over blocks) and the portions of prompts to
        a prefill kernel (tcgen05 with 128 query tokens a block, or mma.sync with 64); otherwise every row is
        a single query of the split kernel, which takes all sizes and both types."""
        rt, g = self.rt, cache.group
        if self.talking:
            # every head's weights need every head's scores: one kernel owns all heads of a query
            # portions of prompts: the tensor-core form where it takes the sizes; single tokens (and everything
            # else): the kernel with a block per token, the key range in pieces when rows are few
            many = step.n_entries - step.n_single
            tc = many > 0 and kernels.attention_talking_mma_fits(rt.dtype, self.nq, self.nkv, self.hd)
            n_rows = step.n_single if tc else T
            if n_rows > 0:
                splits = kernels.attention_talking_splits(n_rows, self.window or 0)
                acc = ml = None
                if splits > 1:   # (rows x pieces never exceeds the number of blocks aimed for)
                    most = kernels.split_target_blocks()
                    acc = rt.scratch.get("talk_part_acc", (most * self.nq * self.hd,), torch.float32)
                    ml = rt.scratch.get("talk_part_ml", (most * self.nq * 2,), torch.float32)
                kernels.attention_talking(q[:n_rows], cache.k, cache.v, o[:n_rows], self.mix, step.positions,
                                          step.entry_of_token, g.block_table, self.window or 0, splits, acc, ml,
                                          sink=self.sink, gate=gate[:n_rows] if gate is not None else None,
                                          status=rt.status)
            if tc:
                kernels.attention_talking_mma(q, cache.k, cache.v, o, self.mix, step.cu_q, step.pos0, g.block_table,
                                              step.n_single, many, step.max_q_len, self.window or 0, sink=self.sink,
                                              gate=gate, status=rt.status)
            return
        mma = rt.dtype == torch.bfloat16 and self.hd in kernels.DECODE_MMA_HEAD_SIZES and not self.float_weights
        extra = {"chunk": self.chunk, "sink": self.sink, "gate": gate} if self.extras else {}
        n_rows = step.n_single if mma else T
        if n_rows > 0:
            per_block = kernels.DECODE_MMA_HEADS_PER_BLOCK if mma else 0
            splits, n_acc, n_ml = kernels.attention_split_plan(n_rows, self.nq, self.nkv, self.hd, per_block)
            part_acc = rt.scratch.get("attn_part_acc", (n_acc,), torch.float32)
            part_ml = rt.scratch.get("attn_part_ml", (n_ml,), torch.float32)
            args = (q, cache.k, cache.v, o, part_acc, part_ml, step.positions, step.entry_of_token, g.block_table,
                    step.n_entries, 0, n_rows, self.window or 0, self.scale, splits)
            if mma and kernels.attention_decode_tma_fits(self.hd, g.page_size):
                # pages arrive as TMA boxes.  Many splits (few rows, long contexts): the last block of a row
                # and head group merges them; few splits: a second small kernel does, during which the
                # output projection already loads its first weights (measured: 2 us a layer either way)
                kernels.attention_decode_tma(*args, status=rt.status, **extra,
                                             merge_counters=rt.merge_counters if splits >= self.MERGE_IN_KERNEL_MIN_SPLITS else None)
            else:
                (kernels.attention_decode_mma if mma else kernels.attention_split)(*args, status=rt.status, **extra)
        if mma and step.n_entries > step.n_single:
            # long portions: 128-token tiles on tcgen05 with the accumulators in tensor memory; short ones
            # (and page sizes a TMA box cannot take): 64-token tiles on mma.sync
            tc = step.max_q_len > 64 and kernels.attention_prefill_tc_fits(self.hd, g.page_size)
            fn = kernels.attention_prefill_tc if tc else kernels.attention_prefill_mma
            fn(q, cache.k, cache.v, o, step.cu_q, step.pos0, g.block_table, step.n_single,
               step.n_entries - step.n_single, step.max_q_len, self.window or 0, self.scale, status=rt.status, **extra)

    MERGE_IN_KERNEL_MIN_SPLITS = 8   # from here on the block that finishes last merges the splits itself
    FUSED_DECODE_MAX_ROWS = 48   # measured: 1.3-2.3 us a layer faster up to 32 rows, 1.6 us slower at 64

    def _fused_decode(self, step, g) -> bool:
        """A step of single tokens only, on the path of the TMA decode kernel (bfloat16, head size 64 or 128,
        a page size it takes), with few enough rows that every block redoing the queries' norm and rotation
        costs less than a kernel of its own."""
        return (not self.float_weights and not self.talking and (self.bias is None or self.own_kv)
                and self.rt.dtype == torch.bfloat16 and self.hd in kernels.DECODE_MMA_HEAD_SIZES
                and kernels.attention_decode_tma_fits(self.hd, g.page_size)
                and step.n_single == step.n_entries == step.n_tokens
                and step.n_tokens <= self.FUSED_DECODE_MAX_ROWS)

    def _convolve(self, qkv, step, state, T):
        """The rows of q | k | v after the short convolution (state: the last taps - 1 rows of each request) and
        the mixing of the values with the first such layer's."""
        rt = self.rt
        C = self.conv_width
        out = rt.scratch.get("attn_qkv_conv", (rt.max_tokens, C), rt.dtype)[:T]
        values = None
        if self.value_mix is not None:
            v_first = rt.scratch.get("attn_v_first:" + str(self.value_mix[1]), (rt.max_tokens, self.nkv * self.v_dim),
                                     rt.dtype)
            values = (self.q_width + self.kv_width, self.nkv, self.hd, self.v_dim, v_first, self.vmix)
        taps = max(self.taps, 1)
        kernels.conv_rows(out, qkv, self.conv_w, taps, C, state if taps > 1 else None, step.entry_of_token, step.cu_q,
                          step.state_slot, step.n_entries, values=values, status=rt.status)
        if taps > 1 and step.n_entries > step.n_single:
            kernels.conv_state_rows(qkv, taps, C, state, step.cu_q, step.state_slot, step.n_single,
                                    step.n_entries - step.n_single)
        return out

    # -- a step ----------------------------------------------------------------
    def forward(self, x, step, cache, state):
        rt = self.rt
        T = x.shape[0]
        nkv_w = self.nkv if self.own_kv else 0
        width = self.in_width if self.own_kv else self.q_width
        qkv = rt.scratch.get("attn_qkv", (rt.max_tokens, width), rt.dtype)[:T]
        rt.linear(qkv, x, self.w_qkv)
        g = cache.group
        gate = qkv[:, self.gate_off:self.gate_off + self.nq] if "gate" in self.names else None
        if self.taps or self.value_mix is not None:
            qkv = self._convolve(qkv, step, state, T)
        o = rt.scratch.get("attn_o", (rt.max_tokens, self.nq, self.hd), rt.dtype)[:T]
        if self._fused_decode(step, g):
            # every row brings one token: the decode attention norms and rotates the queries itself, writes
            # the row's key and value to their page and attends to them: one kernel less in every layer
            splits, n_acc, n_ml = kernels.attention_split_plan(T, self.nq, self.nkv, self.hd,
                                                               kernels.DECODE_MMA_HEADS_PER_BLOCK)
            kernels.attention_decode_tma_fused(
                qkv, cache.k, cache.v, o, rt.scratch.get("attn_part_acc", (n_acc,), torch.float32),
                rt.scratch.get("attn_part_ml", (n_ml,), torch.float32), step.positions, step.entry_of_token,
                g.block_table, step.n_entries, 0, T, self.nq, self.window or 0, self.scale, splits,
                self.q_norm_w, self.k_norm_w, self.norm_eps if self.norm_eps is not None else 1.0,
                self.position.rotary_table(), write_kv=self.own_kv, status=rt.status,
                merge_counters=rt.merge_counters if splits >= self.MERGE_IN_KERNEL_MIN_SPLITS else None,
                bias=self.bias, q_temperature=self.position.query_temperature(), chunk=self.chunk, sink=self.sink,
                gate=gate)
        else:
            q = rt.scratch.get("attn_q", (rt.max_tokens, self.nq, self.hd), rt.dtype)[:T]
            args = (qkv, q, cache.k if self.own_kv else None, cache.v if self.own_kv else None, step.positions,
                    g.slot_map if self.own_kv else None, self.position.rotary_table(), self.q_norm_w, self.k_norm_w,
                    self.norm_eps if self.norm_eps is not None else 1.0, self.nq, nkv_w, self.hd, g.page_size)
            q_temp = self.position.query_temperature()
            if self.bias is not None or q_temp is not None:
                kernels.qkv_bias_rope_kv_write(*args, bias=self.bias, q_temperature=q_temp, status=rt.status)
            else:
                kernels.qk_norm_rope_kv_write(*args, status=rt.status)
            self._attend(q, o, cache, step, T, gate)
        out = rt.scratch.get(self.out_key, (rt.max_tokens, self.hidden), rt.dtype)[:T]
        return rt.linear(out, o.view(T, self.q_width), self.w_o, sink=step.take_sink())
