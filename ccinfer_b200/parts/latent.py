"""Latent attention: keys and values of all heads made from one low-rank vector per token.

With H heads of ``dim`` unrotated and ``rot_dim`` rotated query/key coordinates, value size ``vdim`` and latent
size ``rank``:

    q = Wq x                      [H, dim | rot_dim]
    [c' | kr'] = Wdkv x           c = c' / rms(c') * w_c  (rank),  kr = rot(kr')  (rot_dim, one for all heads)
    k_h = [Wuk_h c | kr],  v_h = Wuv_h c
    s_ij = (q_h,i . k_h,j) * scale  for  0 <= i - j < window;   p = exp(s) / (sum_j exp(s_ij) + exp(sink_h))
    o_h = sigmoid(Wg x)_h * sum_j p_ij v_h,j;   out = Wo [o_1 .. o_H]

The rotation turns the pairs (i, i + rot.dims / 2) of the first ``rot.dims`` rotated coordinates of q and of kr
by position * base^(-2i / rot.dims); with ``interleaved`` the pairs are (2i, 2i + 1) instead, which the kernels see as
the same thing after the rows of Wq's rotated parts and of Wdkv's are permuted alike when they are bound (a score
does not change when q and k are permuted alike).  ``window`` None: every earlier token is seen.  Without a gate
tensor the heads' results are taken as they are.  ``own_kv`` False: the layer has no Wdkv and reads the rows that
another layer of the same latent size, rotated size and rotation left in its cache.

What a token leaves in the cache is the row [c | kr] alone.  Attention runs over those rows: the unrotated part
of a query is carried into the latent space first, (Wuk_h^T q_h) . c = q_h . (Wuk_h c), and the weighted sum of c
comes back out through Wuv_h afterwards (two products per head, batched over the heads).  q, the latent row and
the gate are ONE merged product of x.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import kernels
from ..errors import Unsupported
from .base import CachedTensor, CacheNeed, Mixer, TensorSpec


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class LatentAttention(Mixer):
    kernel_groups = ("latent",)
    def __init__(self, hidden: int, heads: int, dim: int, rot_dim: int, value_dim: int, rank: int, window: int,
                 scale: float, rot_base: float, rot_dims: int, norm_eps: float, names: dict,
                 interleaved: bool = False, own_kv: bool = True):
        """``names``: tensor names under the keys q, dkv, dkv_norm, uk, uv, sink, o and optionally g (the gate)."""
        if window is not None and window <= 0:
            raise Unsupported("a window of keys is > 0 (None: every earlier token)")
        if rot_dims % 2 or not (0 <= rot_dims <= rot_dim):
            raise Unsupported(f"rotation of {rot_dims} of {rot_dim} coordinates: even, at most rot_dim")
        if rank > 1024:
            raise Unsupported(f"latent size {rank}: the attention kernel holds up to 1024 coordinates per warp")
        self.hidden, self.H, self.d, self.r, self.dv, self.R = (int(hidden), int(heads), int(dim), int(rot_dim),
                                                                int(value_dim), int(rank))
        self.window = int(window) if window is not None else None
        self.kernel_window = self.window if self.window is not None else 2 ** 31 - 1   # (what the kernels are told)
        self.scale, self.eps = float(scale), float(norm_eps)
        self.rot_base, self.rot_dims = float(rot_base), int(rot_dims)
        self.interleaved, self.own_kv = bool(interleaved), bool(own_kv)
        self.names = dict(names)
        self.has_gate = "g" in self.names
        # columns of the merged product: q | [c' | kr'] | gate logits, each start a multiple of 8
        self.oq = 0
        self.oc = _pad8(self.H * (self.d + self.r))
        self.og = self.oc + _pad8(self.R + self.r)
        self.in_width = self.og + _pad8(self.H)
        self.rt = None

    def tensor_specs(self):
        n, D, H = self.names, self.hidden, self.H
        specs = [TensorSpec(n["q"], (H * (self.d + self.r), D)),
                 TensorSpec(n["uk"], (H * self.d, self.R)), TensorSpec(n["uv"], (H * self.dv, self.R)),
                 TensorSpec(n["sink"], (H,), role="vector"), TensorSpec(n["o"], (D, H * self.dv))]
        if self.own_kv:
            specs += [TensorSpec(n["dkv"], (self.R + self.r, D)),
                      TensorSpec(n["dkv_norm"], (self.R,), role="vector", init="one_plus_normal")]
        if self.has_gate:
            specs.append(TensorSpec(n["g"], (H, D)))
        return specs

    def cache_need(self):
        return CacheNeed((CachedTensor("latent", (self.R + self.r,), token_axis=0),), self.window)

    def bind(self, rt, fetch):
        self.rt = rt
        n, H = self.names, self.H
        w = torch.zeros((self.in_width, self.hidden), dtype=rt.dtype, device=rt.device)
        # the rotated coordinates in the kernels' order: pair i at places (i, i + rot_dims / 2)
        perm = None
        if self.interleaved and self.rot_dims:
            half = self.rot_dims // 2
            perm = torch.tensor([2 * i for i in range(half)] + [2 * i + 1 for i in range(half)]
                                + list(range(self.rot_dims, self.r)), device=rt.device)
        wq = fetch(n["q"])
        if perm is not None:
            wq = wq.view(H, self.d + self.r, -1).clone()
            wq[:, self.d:] = wq[:, self.d:][:, perm]
            wq = wq.view(H * (self.d + self.r), -1)
        w[self.oq:self.oq + wq.shape[0]] = wq
        if self.own_kv:
            wc = fetch(n["dkv"])
            if perm is not None:
                wc = wc.clone()
                wc[self.R:] = wc[self.R:][perm]
            w[self.oc:self.oc + wc.shape[0]] = wc
        if self.has_gate:
            t = fetch(n["g"])
            w[self.og:self.og + t.shape[0]] = t
        self.w_in = w
        self.norm_w = (fetch(n["dkv_norm"]).float().contiguous() if self.own_kv
                       else torch.ones(self.R, dtype=torch.float32, device=rt.device))
        self.sink = fetch(n["sink"]).float().contiguous()
        # per head: [rank, dim] so that (q_h Wuk_h) is a product with the weights' usual layout [out, in]
        self.w_uk_t = fetch(n["uk"]).view(H, self.d, self.R).transpose(1, 2).contiguous()
        self.w_uv = fetch(n["uv"]).view(H, self.dv, self.R).contiguous()
        self.w_o = fetch(n["o"])
        self.inv_freq = None
        if self.rot_dims:
            i = np.arange(self.rot_dims // 2, dtype=np.float64)
            f = np.power(np.float64(self.rot_base), -2.0 * i / self.rot_dims).astype(np.float32)
            self.inv_freq = torch.from_numpy(f).to(rt.device)

    def forward(self, x, step, cache, state):
        rt = self.rt
        x = rt.rows(x)
        T = x.shape[0]
        H, d, r, R, dv = self.H, self.d, self.r, self.R, self.dv
        g = cache.group
        proj = rt.scratch.get("latent_proj", (rt.max_tokens, self.in_width), rt.dtype)[:T]
        rt.linear(proj, x, self.w_in)
        qa = rt.scratch.get("latent_q", (rt.max_tokens, H, R + r), torch.float32)[:T]
        rows = cache.tensors["latent"]
        kernels.latent_prepare(proj, self.oq, self.oc, self.norm_w, self.inv_freq, self.rot_dims, step.positions,
                               g.slot_map if cache.own else None, rows, qa, H, d, r, R, self.eps, status=rt.status)
        if d > 0:
            qu = proj[:, self.oq:self.oq + H * (d + r)].view(T, H, d + r)[:, :, :d]
            rt.linear_batched(qa[:, :, :R].permute(1, 0, 2), qu.permute(1, 0, 2), self.w_uk_t)
        else:
            qa[:, :, :R].zero_()
        ol = rt.scratch.get("latent_o", (rt.max_tokens, H, R), rt.dtype)[:T]
        gate = proj[:, self.og:self.og + H] if self.has_gate else None
        args = (qa, rows, self.sink, gate, ol, step.cu_q, step.pos0, step.entry_of_token, g.block_table)
        n1, many = step.n_single, step.n_entries - step.n_single
        if kernels.latent_attention_mma_fits(rt.dtype, R, r):
            # tensor cores: the heads are the rows of the products.  The step's single tokens come first; their
            # key ranges are cut into pieces so that a few rows still fill the machine
            if n1 > 0:
                splits = kernels.latent_attention_splits(n1, H, self.kernel_window)
                acc = ml = None
                if splits > 1:
                    most = kernels.latent_attention_splits(1, H, self.kernel_window)   # (rows x pieces is bounded by the target)
                    cap = max(rt.max_entries * H * most, kernels.split_target_blocks() * kernels.LATENT_MMA_ROWS * 2)
                    acc = rt.scratch.get("latent_part_acc", (cap * R,), torch.float32)
                    ml = rt.scratch.get("latent_part_ml", (cap * 2,), torch.float32)
                kernels.latent_attention_mma(*args, 0, n1, 1, g.page_size, self.kernel_window, self.scale, splits, acc, ml,
                                             status=rt.status)
            if many > 0:
                kernels.latent_attention_mma(*args, n1, many, step.max_q_len, g.page_size, self.kernel_window, self.scale,
                                             status=rt.status)
        else:   # the plain kernel: float, and sizes that are multiples of nothing
            if n1 > 0:
                kernels.latent_attention(*args, 0, n1, 1, g.page_size, self.kernel_window, self.scale, status=rt.status)
            if many > 0:
                kernels.latent_attention(*args, n1, many, step.max_q_len, g.page_size, self.kernel_window, self.scale,
                                         status=rt.status)
        o = rt.scratch.get("latent_v", (rt.max_tokens, H, dv), rt.dtype)[:T]
        rt.linear_batched(o.permute(1, 0, 2), ol.permute(1, 0, 2), self.w_uv)
        out = rt.scratch.get(self.out_key, (rt.max_tokens, self.hidden), rt.dtype)[:T]
        return rt.linear(out, o.view(T, H * dv), self.w_o)
