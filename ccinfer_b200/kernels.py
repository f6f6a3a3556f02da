"""Python face of the CUDA kernels: one function per launcher of ``csrc``.

The shared object is loaded with ctypes; tensors are passed as raw device
pointers and every launch goes to torch's current CUDA stream, so the kernels
take part in stream capture like any other work.  A launcher that refuses its
arguments or whose launch fails raises; nothing falls back to another
implementation.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_size_t, c_void_p

import torch

from .csrc import build as _build
from .errors import ExtensionMissing, InvalidArgument, Unsupported

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

ST_BAD_TOKEN, ST_BAD_SLOT, ST_BAD_PAGE, ST_BAD_ROW, ST_WAIT_TIMEOUT = 1, 2, 4, 8, 16
STATUS_TEXT = {
    ST_BAD_TOKEN: "a token id outside the vocabulary",
    ST_BAD_SLOT: "a cache slot outside the pool",
    ST_BAD_PAGE: "a block-table entry outside the pool where a key was needed",
    ST_BAD_ROW: "a row index outside the batch",
    ST_WAIT_TIMEOUT: "a bounded wait inside a kernel gave up",
}

_lock = threading.Lock()
_libs = {}

_SIGNATURES = {
    "ccb_embed_gather": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                         c_void_p],
    "ccb_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "ccb_gemm_tc_swiglu_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                c_void_p],
    "ccb_gemm_tc_glu_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                             c_float, c_void_p, c_void_p],
    "ccb_gemm_fewrows_glu_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_float, c_float, c_float, c_void_p, c_void_p],
    "ccb_gemm_tc_pair_glu_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_float, c_float, c_int, c_void_p, c_void_p],
    "ccb_gemm_fewrows_set_stages": [c_int],
    "ccb_gemm_fewrows_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_void_p, c_void_p],
    "ccb_gemm_fewrows_blocks": [c_int],
    "ccb_gemm_fewrows_norm_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_void_p, c_int, c_float, c_float, c_void_p, c_int, c_void_p, c_void_p,
                                   c_void_p, c_void_p],
    "ccb_gemm_tc_swiglu_scaled_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_void_p, c_int, c_float, c_float, c_void_p, c_void_p],
    "ccb_residual_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                             c_int, c_void_p, c_void_p],
    "ccb_embed_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int,
                          c_void_p, c_int, c_void_p, c_void_p],
    "ccb_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    "ccb_qk_norm_rope_kv_write": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_void_p, c_void_p],
    "ccb_qkv_bias_rope_kv_write": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_void_p, c_float, c_int, c_void_p, c_void_p],
    "ccb_postnorm_residual": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p, c_float,
                              c_int, c_int, c_int, c_void_p],
    "ccb_clamped_glu": [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_float, c_int, c_void_p],
    "ccb_delta_prepare": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
                          c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p],
    "ccb_conv_state_update": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int,
                              c_int, c_int, c_int, c_int, c_int, c_void_p],
    "ccb_delta_recurrence": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "ccb_gated_head_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_int,
                               c_int, c_void_p],
    "ccb_gated_linear_recurrence": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_int, c_int, c_int, c_int, c_int, c_void_p],
    "ccb_gla_prepare": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p],
    "ccb_latent_prepare": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                           c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "ccb_latent_attention": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                             c_int, c_void_p, c_void_p],
    "ccb_latent_attention_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "ccb_latent_attention_mma_fits": [c_int, c_int],
    "ccb_moe_route": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                      c_int, c_int, c_int, c_float, c_void_p],
    "ccb_moe_dense_glu_act": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_void_p],
    "ccb_conv_rows": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p,
                      c_void_p],
    "ccb_conv_state_rows": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                            c_void_p],
    "ccb_attention_split_ex": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                               c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "ccb_moe_dense_act": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "ccb_moe_sort": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                     c_void_p, c_void_p, c_void_p],
    "ccb_moe_route_sort": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                           c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                           c_void_p],
    "ccb_moe_grouped": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_void_p, c_void_p,
                        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "ccb_moe_gather_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "ccb_moe_grouped_tc": [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "ccb_moe_combine": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "ccb_scaled_residual": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_void_p],
    "ccb_concat_cast": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "ccb_add_row": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "ccb_gelu_gate_rows": [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                           c_int, c_void_p, c_void_p],
    "ccb_gemm_f32_batched": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_longlong,
                             c_longlong, c_longlong, c_int, c_void_p],
    "ccb_gemm_bf16_batched": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_longlong, c_longlong, c_longlong, c_int, c_int, c_void_p],
    "ccb_paged_attention_generic": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                    c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                    c_void_p, c_void_p],
    "ccb_attention_split": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                            c_int, c_void_p, c_void_p],
    # (the four arguments before the status word: chunk, sink, gate, gate_stride)
    "ccb_attention_decode_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "ccb_attention_decode_tma": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_float, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "ccb_attention_decode_tma_fused": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_float, c_void_p, c_int,
                                       c_void_p, c_float, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                       c_void_p, c_void_p],
    "ccb_attention_prefill_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                     c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "ccb_attention_prefill_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                 c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "ccb_gemm_f32": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "ccb_cublas_create": [ctypes.POINTER(c_void_p)],
    "ccb_cublas_destroy": [c_void_p],
    "ccb_cublas_set_workspace": [c_void_p, c_void_p, c_size_t],
    "ccb_gemm_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                      c_void_p],
    "ccb_gemm_skinny_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_void_p],
    "ccb_gemm_tc_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_void_p, c_void_p, c_void_p, c_void_p],
    "ccb_gemm_tc_pair_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_void_p, c_void_p],
    "ccb_init_random": [c_void_p, c_longlong, c_int, ctypes.c_ulonglong, ctypes.c_ulonglong, c_float, c_int, c_void_p],
    "ccb_ssm_prepare": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                        c_int, c_int, c_int, c_void_p],
    "ccb_conv_state_shift": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_void_p],
    "ccb_gemm_fewrows_relu2_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                    c_void_p, c_void_p],
    "ccb_ssm_gate_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                          c_int, c_float, c_int, c_void_p],
    "ccb_ssm_recurrence": [c_void_p] * 9 + [c_int] * 5 + [c_void_p],
    "ccb_attention_talking_fits": [c_int, c_int, c_int],
    "ccb_attention_talking": [c_void_p] * 10 + [c_int] * 9 + [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "ccb_attention_talking_mma_fits": [c_int, c_int, c_int],
    "ccb_attention_talking_mma": [c_void_p] * 8 + [c_int] * 10 + [c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "ccb_embed_pair": [c_void_p] * 10 + [c_float] + [c_int] * 9 + [c_void_p, c_int, c_void_p, c_void_p],
    "ccb_relu_squared": [c_void_p, c_void_p, c_longlong, c_int, c_void_p],
    "ccb_scaled_sum": [c_void_p, c_void_p, c_void_p, c_float, c_float, c_longlong, c_int, c_void_p],
    "ccb_sample_rows": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                        c_int, c_void_p, c_void_p, c_int, c_void_p],
}


_pdl = None          # what set_pdl was last told: a family that is loaded later is told the same
_group_of = {}       # exported function -> kernel family


def _load(group: str):
    """The loaded shared object of a kernel family (built at the first call)."""
    with _lock:
        if group in _libs:
            return _libs[group]
        path = _build.library_path(group)
        try:
            handle = ctypes.CDLL(path)
        except OSError as e:
            raise ExtensionMissing(f"cannot load {path}: {e}") from e
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is not None:
                fn.argtypes = argtypes
                fn.restype = c_int
        handle.ccb_set_pdl.argtypes = [c_int]
        handle.ccb_set_pdl.restype = c_int
        if _pdl is not None:
            handle.ccb_set_pdl(_pdl)
        _libs[group] = handle
        return handle


class _Kernels:
    """All kernel families as one object: ``lib().ccb_name`` finds the family that exports ``ccb_name`` (from the
    sources' text), builds and loads it if this is its first use, and hands the function out.  A model therefore
    compiles the families whose kernels it launches and no others."""

    def __getattr__(self, name):
        if not _group_of:
            for group in _build.KERNEL_GROUPS:
                for fn in _build.exported_functions(group):
                    _group_of.setdefault(fn, group)
        group = _group_of.get(name)
        if group is None:
            raise AttributeError(f"no kernel family exports {name!r}")
        fn = getattr(_load(group), name)
        setattr(self, name, fn)   # (found once)
        return fn


_kernels = _Kernels()


def lib(group: str = None):
    """The kernels (see ``_Kernels``), or with ``group`` the loaded shared object of that one family."""
    if group is not None:
        return _load(group)
    _load("base")   # (what every model needs: a missing compiler shows here, before anything else happens)
    return _kernels


def prepare(groups) -> None:
    """Builds (side by side) and loads the kernel families named, e.g. those a model's parts say they launch
    (``Part.kernel_groups``), so that the first step does not build them one after another as it meets them."""
    wanted = [g for g in dict.fromkeys(["base"] + list(groups)) if g not in _libs]
    if len(wanted) > 1:
        _build.build_groups(wanted)
    for g in wanted:
        _load(g)


def set_pdl(on) -> None:
    """Launch the library's kernels so that each may start while its predecessor finishes (programmatic
    dependent launch); every kernel waits for its predecessor before it reads what that one wrote."""
    global _pdl
    _pdl = int(on)
    with _lock:
        loaded = list(_libs.values())
    for handle in loaded:
        handle.ccb_set_pdl(_pdl)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class _Counters:
    """Launches since import: ``own`` = kernels of this package, ``library`` = cuBLAS products."""
    own = 0
    library = 0


counters = _Counters()


def _check(code: int, what: str) -> None:
    if code == 0:
        if what == "gemm_bf16":
            counters.library += 1
        elif not what.startswith("cublas"):
            counters.own += 1
        return
    if code == -2:
        raise Unsupported(f"{what}: a size outside what the kernel takes")
    if code == -3:
        raise Unsupported(f"{what}: element type not supported")
    if code == -4:
        raise InvalidArgument(f"{what}: a required argument is missing")
    if code >= 1000:
        raise RuntimeError(f"{what}: cuBLAS status {code - 1000}")
    raise RuntimeError(f"{what}: CUDA error {code}")


def _p(t):
    return 0 if t is None else t.data_ptr()


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise Unsupported(f"element type {t.dtype} is not supported by the kernels") from None


def _cuda(*tensors):
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise InvalidArgument("kernels take contiguous CUDA tensors")


def status_message(word: int) -> str:
    return "; ".join(text for bit, text in STATUS_TEXT.items() if word & bit) or "no fault"


# ---------------------------------------------------------------------------------------------
def embed_gather(h: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, status=None, pending=None) -> None:
    """h[t, :] = float(table[ids[t], :]); h is the float residual stream [T, D].

    With ``pending`` (int32 [slots]) an id of -1 - s stands for pending[s]: the token that sample_rows
    last stored for request slot s."""
    _cuda(h, table, ids, status, pending)
    T, D = h.shape
    assert h.dtype == torch.float32 and ids.dtype == torch.int32 and table.shape[1] == D and ids.numel() >= T
    assert pending is None or pending.dtype == torch.int32
    _check(lib().ccb_embed_gather(_p(h), _p(table), _p(ids), T, D, table.shape[0], _dt(table), _p(pending),
                                  0 if pending is None else pending.numel(), _p(status), _stream()), "embed_gather")


def embed_rmsnorm(y, h, table, ids, w, eps: float, status=None, pending=None) -> None:
    """embed_gather and the norm of the rows it wrote in one pass: h[t, :] = float(table[ids[t], :]) and
    y[t, :] = RMSNorm(h[t, :]) * w (y and table in the storage type, w float)."""
    _cuda(y, h, table, ids, w, status, pending)
    T, D = h.shape
    assert h.dtype == torch.float32 and ids.dtype == torch.int32 and table.shape[1] == D and ids.numel() >= T
    assert y.shape == (T, D) and y.dtype == table.dtype and w.dtype == torch.float32 and w.numel() == D
    assert h.is_contiguous() and y.is_contiguous() and table.is_contiguous()
    assert pending is None or pending.dtype == torch.int32
    _check(lib().ccb_embed_rmsnorm(_p(y), _p(h), _p(table), _p(ids), _p(w), T, D, table.shape[0], float(eps),
                                   _dt(table), _p(pending), 0 if pending is None else pending.numel(), _p(status),
                                   _stream()), "embed_rmsnorm")


def silu_mul(act: torch.Tensor, gate_up: torch.Tensor, block: int = 0) -> None:
    """act[t, f] = silu(gate[t, f]) * up[t, f] for gate_up[t, :] = [all gate | all up] (block = 0) or in
    blocks of ``block`` gate columns followed by the ``block`` up columns of the same channels."""
    _cuda(act, gate_up)
    T, F = act.shape
    assert gate_up.shape == (T, 2 * F) and act.dtype == gate_up.dtype
    _check(lib().ccb_silu_mul(_p(act), _p(gate_up), T, F, int(block), _dt(act), _stream()), "silu_mul")


SWIGLU_BLOCK = 64   # rows of gate, then of up, in a weight matrix laid out for gemm_tc_swiglu_bf16


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int) -> torch.Tensor:
    """[2F, D]: ``block`` rows of gate, the ``block`` rows of up for the same channels, and so on."""
    F, D = gate.shape
    assert up.shape == (F, D) and F % block == 0
    return torch.cat([gate.view(F // block, block, D), up.view(F // block, block, D)], dim=1).reshape(2 * F, D).contiguous()


def gemm_tc_swiglu_bf16(act, a, w, status=None) -> None:
    """act[M, F] = silu(a Wg^T) * (a Wu^T) in one tensor-core kernel; w [2F, K] interleaved in blocks of
    SWIGLU_BLOCK rows (interleave_gate_up), M <= 16, F a multiple of 64."""
    _cuda(act, a, w, status)
    assert act.dtype == a.dtype == w.dtype == torch.bfloat16
    M, K = a.shape
    F = w.shape[0] // 2
    assert w.shape == (2 * F, K) and act.shape == (M, F) and a.stride(1) == w.stride(1) == act.stride(1) == 1
    _check(lib().ccb_gemm_tc_swiglu_bf16(_p(act), _p(a), _p(w), M, F, K, a.stride(0), w.stride(0), act.stride(0),
                                         _p(status), _stream()), "gemm_tc_swiglu_bf16")


def gemm_glu_bf16(act, a, w, limit: float, alpha: float, shift: float, kind: str, status=None) -> None:
    """act[M, F] = glu(a Wg^T, a Wu^T) with the clamped activation of ``clamped_glu`` as the epilogue of the
    product, w [2F, K] interleaved in blocks of SWIGLU_BLOCK rows.  ``kind``: "tc" (tcgen05, M <= 16),
    "fewrows" (TMA ring, M <= 16) or "pair" (tcgen05 on pairs of SMs, many rows)."""
    _cuda(w, status)
    assert a.dtype == w.dtype == act.dtype == torch.bfloat16 and act.is_cuda and a.is_cuda
    M, K = a.shape
    F = act.shape[1]
    assert w.shape == (2 * F, K) and act.shape[0] == M and F % SWIGLU_BLOCK == 0
    assert a.stride(1) == 1 and w.stride(1) == 1 and act.stride(1) == 1
    args = (float(limit), float(alpha), float(shift))
    if kind == "tc":
        rc = lib().ccb_gemm_tc_glu_bf16(_p(act), _p(a), _p(w), M, F, K, a.stride(0), w.stride(0), act.stride(0),
                                        *args, _p(status), _stream())
    elif kind == "fewrows":
        rc = lib().ccb_gemm_fewrows_glu_bf16(_p(act), _p(a), _p(w), M, 2 * F, K, a.stride(0), w.stride(0),
                                             act.stride(0), _dt(act), *args, _p(status), _stream())
    else:
        rc = lib().ccb_gemm_tc_pair_glu_bf16(_p(act), _p(a), _p(w), M, 2 * F, K, a.stride(0), w.stride(0),
                                             act.stride(0), *args, sm_count(), _p(status), _stream())
    _check(rc, "gemm_glu_bf16")


def gemm_tc_swiglu_scaled_bf16(act, a, w, ssq, parts: int, dim: int, eps: float, status=None) -> None:
    """gemm_tc_swiglu_bf16 whose token rows still lack the factor of their RMSNorm: token t of both products is
    multiplied by 1 / sqrt(sum_p ssq[t, p] / dim + eps) before the activation (ssq float [16, parts])."""
    _cuda(act, a, w, ssq, status)
    assert act.dtype == a.dtype == w.dtype == torch.bfloat16 and ssq.dtype == torch.float32
    M, K = a.shape
    F = w.shape[0] // 2
    assert w.shape == (2 * F, K) and act.shape == (M, F) and a.stride(1) == w.stride(1) == act.stride(1) == 1
    assert ssq.is_contiguous() and ssq.numel() >= parts * 16
    _check(lib().ccb_gemm_tc_swiglu_scaled_bf16(_p(act), _p(a), _p(w), M, F, K, a.stride(0), w.stride(0),
                                                act.stride(0), _p(ssq), int(parts), float(dim), float(eps),
                                                _p(status), _stream()), "gemm_tc_swiglu_scaled_bf16")


def residual_rmsnorm(y, h, delta, w, eps: float, row_idx=None, n_rows=None, status=None) -> None:
    """y = RMSNorm(h + delta) * w, and h <- h + delta when no rows are picked.

    h float [T, D]; delta (optional) and y in the storage type; w float [D].
    With ``row_idx`` (int32 [R]) only those rows of h are normed, into y [R, D].
    """
    _cuda(y, h, delta, w, row_idx, status)
    D = h.shape[1]
    rows = y.shape[0] if n_rows is None else n_rows
    assert h.dtype == torch.float32 and w.dtype == torch.float32 and w.numel() == D and y.shape[1] == D
    assert delta is None or (delta.dtype == y.dtype and delta.shape[1] == D)
    _check(lib().ccb_residual_rmsnorm(_p(y), _p(h), _p(delta), _p(w), _p(row_idx), rows, h.shape[0], D,
                                      float(eps), _dt(y), _p(status), _stream()), "residual_rmsnorm")


def rmsnorm(y, x, w, eps: float) -> None:
    """Plain RMSNorm over the last axis of a contiguous tensor; w float."""
    _cuda(y, x, w)
    D = x.shape[-1]
    assert w.dtype == torch.float32 and w.numel() == D and y.dtype == x.dtype and y.shape == x.shape
    _check(lib().ccb_rmsnorm(_p(y), _p(x), _p(w), x.numel() // D, D, float(eps), _dt(x), _stream()), "rmsnorm")


def qk_norm_rope_kv_write(qkv, q_out, k_cache, v_cache, positions, slot_map, inv_freq, q_w, k_w, eps,
                          nq: int, nkv: int, hd: int, page_size: int, status=None) -> None:
    """Head norms, rotation and cache write in one pass over qkv [T, (nq + 2 nkv) hd].

    q goes to q_out [T, nq, hd]; k and v go to their caches [pages, nkv, page, hd]
    at slot_map[t] (a negative slot skips the write).  inv_freq, q_w, k_w may
    be None to leave that step out; nkv = 0 handles q alone.
    """
    _cuda(qkv, q_out, k_cache, v_cache, positions, slot_map, inv_freq, q_w, k_w, status)
    T = q_out.shape[0]
    assert qkv.shape[0] >= T and qkv.shape[1] >= (nq + 2 * nkv) * hd and qkv.dtype == q_out.dtype
    num_slots = 0
    if nkv > 0:
        assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
        assert k_cache.shape[1:] == (nkv, page_size, hd) and v_cache.shape == k_cache.shape
        num_slots = k_cache.shape[0] * page_size
    _check(lib().ccb_qk_norm_rope_kv_write(_p(qkv), qkv.stride(0), _p(q_out), _p(k_cache), _p(v_cache),
                                           _p(positions), _p(slot_map), _p(inv_freq), _p(q_w), _p(k_w),
                                           float(eps), T, nq, nkv, hd, page_size, num_slots, _dt(qkv),
                                           _p(status), _stream()), "qk_norm_rope_kv_write")


def qkv_bias_rope_kv_write(qkv, q_out, k_cache, v_cache, positions, slot_map, inv_freq, q_w, k_w, eps,
                           nq: int, nkv: int, hd: int, page_size: int, bias=None, q_temperature=None,
                           status=None) -> None:
    """qk_norm_rope_kv_write for projections with biases and queries with a temperature.

    ``bias`` float [(nq + 2 nkv) * hd] is added to the rows of qkv before anything else;
    ``q_temperature = (coef, every)``: q *= 1 + coef * ln(floor((pos + 1) / every) + 1) after the rotation."""
    _cuda(qkv, q_out, k_cache, v_cache, positions, slot_map, inv_freq, q_w, k_w, bias, status)
    T = q_out.shape[0]
    assert qkv.shape[0] >= T and qkv.shape[1] >= (nq + 2 * nkv) * hd and qkv.dtype == q_out.dtype
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == (nq + 2 * nkv) * hd)
    num_slots = 0
    if nkv > 0:
        assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
        assert k_cache.shape[1:] == (nkv, page_size, hd) and v_cache.shape == k_cache.shape
        num_slots = k_cache.shape[0] * page_size
    coef, every = q_temperature if q_temperature is not None else (0.0, 0)
    _check(lib().ccb_qkv_bias_rope_kv_write(_p(qkv), qkv.stride(0), _p(q_out), _p(k_cache), _p(v_cache),
                                            _p(positions), _p(slot_map), _p(inv_freq), _p(q_w), _p(k_w),
                                            float(eps), T, nq, nkv, hd, page_size, num_slots, _dt(qkv), _p(bias),
                                            float(coef), int(every), _p(status), _stream()),
           "qkv_bias_rope_kv_write")


def postnorm_residual(h, delta, w_post, mult: float, eps_post: float, add=None, y=None, w_next=None,
                      eps_next: float = 0.0) -> None:
    """h += mult * RMSNorm(delta; w_post) [+ add]; with ``w_next``, y = RMSNorm(h; w_next) in the same pass; with
    ``y`` alone, y = h in the storage type (for a sublayer that reads the stream itself).

    h and add float [T, D]; delta and y in the storage type; the weights float [D].  ``delta`` None: only the
    addition of ``add`` and/or the second norm."""
    _cuda(h, delta, w_post, add, y, w_next)
    T, D = h.shape
    assert h.dtype == torch.float32 and (delta is None or (delta.shape == (T, D) and w_post.numel() == D))
    assert add is None or (add.dtype == torch.float32 and add.shape[1] == D and add.shape[0] >= T)
    assert w_next is None or (y is not None and y.shape == (T, D) and w_next.numel() == D)
    assert delta is None or y is None or delta.dtype == y.dtype
    ref = delta if delta is not None else y
    _check(lib().ccb_postnorm_residual(_p(y), _p(h), _p(delta), _p(w_post), float(mult), float(eps_post), _p(add),
                                       _p(w_next), float(eps_next), T, D, _dt(ref) if ref is not None else F32,
                                       _stream()), "postnorm_residual")


def clamped_glu(act, gate_up, block: int, limit: float, alpha: float, up_shift: float) -> None:
    """act = g * sigmoid(alpha g) * (u + up_shift) with g = min(gate, limit), u = clamp(up, -limit, limit);
    the layouts of gate_up are those of ``silu_mul``."""
    _cuda(act, gate_up)
    T, F = act.shape
    assert gate_up.shape == (T, 2 * F) and act.dtype == gate_up.dtype
    _check(lib().ccb_clamped_glu(_p(act), _p(gate_up), T, F, int(block), float(limit), float(alpha),
                                 float(up_shift), _dt(act), _stream()), "clamped_glu")


def delta_prepare(proj, offsets, a, conv_w, taps: int, conv_state, A_log, dt_bias, entry_of_token, cu_q, state_slot,
                  qn, kn, vv, gg, bb, G: int, H: int, dk: int, dv: int, q_mult: float, unit_eps: float) -> None:
    """The inputs of the gated delta rule from the projections' rows: convolution + silu of q, k, v (with the
    request's convolution state before the portion), unit q and k per head (q times ``q_mult``),
    beta = sigmoid(b), decay = exp(-exp(A_log) softplus(a + dt_bias)); outputs float.  ``offsets`` = the first
    columns of q, k, v, b in ``proj``; ``conv_w`` [taps, channels of q|k|v]."""
    _cuda(conv_w, conv_state, A_log, dt_bias, entry_of_token, cu_q, state_slot, qn, kn, vv, gg, bb)
    T = qn.shape[0]
    assert proj.stride(1) == 1 and a.stride(1) == 1 and proj.dtype == a.dtype == conv_state.dtype
    assert conv_w.dtype == torch.float32 and conv_w.shape == (taps, 2 * G * dk + H * dv)   # tap-major
    oq, ok, ov, ob = offsets
    _check(lib().ccb_delta_prepare(_p(proj), proj.stride(0), oq, ok, ov, ob, _p(a), a.stride(0), _p(conv_w), taps,
                                   _p(conv_state), _p(A_log), _p(dt_bias), _p(entry_of_token), _p(cu_q),
                                   _p(state_slot), _p(qn), _p(kn), _p(vv), _p(gg), _p(bb), T, G, H, dk, dv,
                                   float(q_mult), float(unit_eps), _dt(proj), _stream()), "delta_prepare")


def conv_state_update(proj, offsets, conv_state, taps: int, cu_q, state_slot, n_entries: int, G: int, H: int,
                      dk: int, dv: int) -> None:
    """The last taps - 1 rows of q|k|v of each request's portion become its convolution state."""
    _cuda(conv_state, cu_q, state_slot)
    oq, ok, ov, _ = offsets
    _check(lib().ccb_conv_state_update(_p(proj), proj.stride(0), oq, ok, ov, _p(conv_state), taps, _p(cu_q),
                                       _p(state_slot), n_entries, G, H, dk, dv, _dt(proj), _stream()),
           "conv_state_update")


def conv_rows(out, rows, w, taps: int, C: int, state, entry_of_token, cu_q, state_slot, n_entries: int,
              values=None, status=None) -> None:
    """A short causal convolution over time on the first ``C`` columns of a step's rows: out[t, c] = sum_j
    w[j, c] * u[t - taps + 1 + j, c] over the request's rows in order, those before the step's first one taken from
    ``state`` [slots, taps - 1, C] (compute type; zeros for a new request).  ``w`` float [taps, C] (tap-major), or None
    with taps 1 for no convolution.  A request that brings one token has its state moved on here; for the others call
    ``conv_state_rows`` afterwards.  ``values`` = (v_off, heads, head_size, real_size, v_first, lam): the columns
    from v_off on are value heads of ``head_size`` coordinates of which ``real_size`` are real; with ``lam`` None
    the results are also left in ``v_first`` [T, heads * real_size], else out = (1 - lam) out + lam v_first
    (``lam`` a float tensor of one element)."""
    _cuda(w, state, entry_of_token, cu_q, state_slot, status)
    T = rows.shape[0]
    assert rows.dtype == out.dtype and rows.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == T
    assert w is None or (w.dtype == torch.float32 and w.shape == (taps, C))
    assert state is None or (state.dtype == rows.dtype and tuple(state.shape[1:]) == (taps - 1, C))
    vmode, v_off, vh, vhd, vd, v_first, lam = 0, 0, 0, 0, 0, None, None
    if values is not None:
        v_off, vh, vhd, vd, v_first, lam = values
        vmode = 1 if lam is None else 2
        _cuda(v_first, lam)
        assert v_first.dtype == rows.dtype and v_first.shape[0] >= T and v_first[0].numel() == vh * vd
        assert lam is None or (lam.dtype == torch.float32 and lam.numel() == 1)
    _check(lib().ccb_conv_rows(_p(rows), rows.stride(0), _p(out), out.stride(0), _p(w), int(taps), int(C), _p(state),
                               _p(entry_of_token), _p(cu_q), _p(state_slot), T, int(n_entries),
                               state.shape[0] if state is not None else 0, int(v_off), int(vh), int(vhd), int(vd),
                               _p(v_first), _p(lam), vmode, _dt(rows), _p(status), _stream()), "conv_rows")


def conv_state_rows(rows, taps: int, C: int, state, cu_q, state_slot, entry0: int, n_entries: int) -> None:
    """After ``conv_rows``: the last taps - 1 rows of every request among the entries entry0 .. entry0 + n_entries
    - 1 that brought more than one token become its state."""
    _cuda(state, cu_q, state_slot)
    assert state.dtype == rows.dtype and rows.stride(1) == 1 and tuple(state.shape[1:]) == (taps - 1, C)
    _check(lib().ccb_conv_state_rows(_p(rows), rows.stride(0), int(taps), int(C), _p(state), _p(cu_q), _p(state_slot),
                                     int(entry0), int(n_entries), state.shape[0], _dt(rows), _stream()),
           "conv_state_rows")


def delta_recurrence(qn, kn, vv, gg, bb, state, out, cu_q, state_slot, n_entries: int, G: int, H: int, dk: int,
                     dv: int) -> None:
    """The gated delta rule over each request's tokens of the step, from and into ``state``
    [slots, H, dv, dk] (float); out float [T, H, dv]."""
    _cuda(qn, kn, vv, gg, bb, state, out, cu_q, state_slot)
    assert state.dtype == torch.float32 and state.shape[1:] == (H, dv, dk) and out.dtype == torch.float32
    _check(lib().ccb_delta_recurrence(_p(qn), _p(kn), _p(vv), _p(gg), _p(bb), _p(state), _p(out), _p(cu_q),
                                      _p(state_slot), n_entries, G, H, dk, dv, _stream()), "delta_recurrence")


def gated_head_rmsnorm(y, o, gate, w, H: int, dv: int, eps: float, silu_gate: bool = False) -> None:
    """y[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w * sigmoid(gate[t, h, :]); o float, gate and y storage type.
    ``silu_gate``: the factor is gate * sigmoid(gate) instead."""
    _cuda(y, o, w)
    T = y.shape[0]
    assert o.dtype == torch.float32 and w.dtype == torch.float32 and w.numel() == dv and gate.stride(1) == 1
    assert gate.dtype == y.dtype
    _check(lib().ccb_gated_head_rmsnorm(_p(y), _p(o), _p(gate), gate.stride(0), _p(w), T, H, dv, float(eps),
                                        1 if silu_gate else 0, _dt(y), _stream()), "gated_head_rmsnorm")


def gated_linear_recurrence(qn, kn, vv, gg, state, out, cu_q, state_slot, n_entries: int, H: int, dk: int,
                            dv: int) -> None:
    """S <- diag(g_t) S + k_t v_t^T, out_t = S^T q_t over each request's tokens of the step, from and into
    ``state`` [slots, H, dv, dk] (float); the rows float [T, H, dk] (q, k, g) and [T, H, dv] (v, out)."""
    _cuda(qn, kn, vv, gg, state, out, cu_q, state_slot)
    assert state.dtype == torch.float32 and state.shape[1:] == (H, dv, dk) and out.dtype == torch.float32
    assert qn.dtype == kn.dtype == vv.dtype == gg.dtype == torch.float32
    _check(lib().ccb_gated_linear_recurrence(_p(qn), _p(kn), _p(vv), _p(gg), _p(state), _p(out), _p(cu_q),
                                             _p(state_slot), n_entries, H, H, dk, dv, _stream()),
           "gated_linear_recurrence")


def gla_prepare(proj, offsets, a, bias, qn, kn, vv, gg, H: int, dk: int, dv: int, q_mult: float, tau: float) -> None:
    """The float rows of the gated linear recurrence from the projections' rows: q * q_mult, k, v, and the decay
    sigmoid(a + bias)^(1 / tau) per head and key channel.  ``offsets``: first columns of q, k, v in ``proj``."""
    _cuda(bias, qn, kn, vv, gg)
    T = qn.shape[0]
    assert proj.stride(1) == 1 and a.stride(1) == 1 and proj.dtype == a.dtype
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == H * dk)
    oq, ok, ov = offsets
    _check(lib().ccb_gla_prepare(_p(proj), proj.stride(0), oq, ok, ov, _p(a), a.stride(0), _p(bias), _p(qn), _p(kn),
                                 _p(vv), _p(gg), T, H, dk, dv, float(q_mult), float(tau), _dt(proj), _stream()),
           "gla_prepare")


def latent_prepare(proj, oq: int, oc: int, w, inv_freq, rot_dims: int, positions, slot_map, cache, qa, H: int,
                   d: int, r: int, R: int, eps: float, status=None) -> None:
    """The cache rows and the rotated query parts of latent attention from the projections' rows.

    ``proj`` [T, >=]: H query heads of [d | r] from column ``oq``, the latent row [R | r] from ``oc``.  Token t's
    cache row (``cache`` viewed as [slots, R + r], slot_map[t]; a negative slot skips it) gets
    [x / rms(x) * w | rot(x')]; ``qa`` float [T, H, R + r] gets rot(q's last r) in the last r places of each head.
    The rotation turns the pairs (i, i + rot_dims / 2) of the first rot_dims coordinates by pos * inv_freq[i]."""
    _cuda(w, inv_freq, positions, slot_map, cache, qa, status)
    T = qa.shape[0]
    assert proj.stride(1) == 1 and proj.dtype == cache.dtype and qa.dtype == torch.float32
    assert qa.shape == (T, H, R + r) and w.dtype == torch.float32 and w.numel() == R
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() >= rot_dims // 2)
    assert cache.shape[-1] == R + r
    _check(lib().ccb_latent_prepare(_p(proj), proj.stride(0), oq, oc, _p(w), _p(inv_freq), rot_dims, _p(positions),
                                    _p(slot_map), _p(cache), cache.numel() // (R + r), _p(qa), T, H, d, r, R,
                                    float(eps), _dt(proj), _p(status), _stream()), "latent_prepare")


def latent_attention(qa, cache, sink, gate, out, cu_q, pos0, entry_of_token, block_table, entry0: int, n_entries: int,
                     max_q: int, page_size: int, window: int, scale: float, status=None) -> None:
    """Attention of the step's entries entry0 .. entry0 + n_entries - 1 (none with more than ``max_q`` tokens) over
    the cached rows [c | kr] (``cache`` [pages, page_size, R + r]): every head of ``qa`` float [T, H, R + r] reads
    the same rows; a query at position p sees p - window + 1 .. p; the softmax has one more term exp(sink[h]);
    out[t, h, :] = sigmoid(gate[t, h]) * sum_j p_j c_j, [T, H, R] in the storage type."""
    _cuda(qa, cache, sink, out, cu_q, pos0, entry_of_token, block_table, status)
    T, H, W = qa.shape
    R = out.shape[2]
    assert out.shape == (T, H, R) and cache.shape[1:] == (page_size, W) and out.dtype == cache.dtype
    assert gate is None or (gate.dtype == out.dtype and gate.stride(1) == 1)   # None: no gate
    assert sink.dtype == torch.float32 and sink.numel() == H and qa.dtype == torch.float32
    _check(lib().ccb_latent_attention(_p(qa), _p(cache), _p(sink), _p(gate), gate.stride(0) if gate is not None else 0, _p(out), _p(cu_q),
                                      _p(pos0), _p(entry_of_token), _p(block_table), block_table.stride(0), entry0,
                                      n_entries, max_q, H, R, W - R, page_size, cache.shape[0], int(window),
                                      float(scale), _dt(out), _p(status), _stream()), "latent_attention")


def latent_attention_mma_fits(dtype, R: int, r: int) -> bool:
    """Whether the tensor-core form of latent attention takes these sizes."""
    return dtype == torch.bfloat16 and R % 16 == 0 and r % 16 == 0 and 0 < R <= 512


LATENT_MMA_KEYS = 32       # keys a block of the tensor-core form takes at a time
LATENT_MMA_ROWS = 16       # (query, head) rows of a block


def latent_attention_splits(n_rows: int, H: int, window: int) -> int:
    """Into how many pieces the key range of single-token rows is cut: enough blocks for two per SM, at most one
    piece per 32 keys.  It depends on the number of rows only, so a step of a given size launches one grid."""
    groups = -(-H // min(LATENT_MMA_ROWS, H))
    most = min(64, -(-window // LATENT_MMA_KEYS) + 1)
    return max(1, min(most, split_target_blocks() // max(1, n_rows * groups)))


def latent_attention_mma(qa, cache, sink, gate, out, cu_q, pos0, entry_of_token, block_table, entry0: int,
                         n_entries: int, max_q: int, page_size: int, window: int, scale: float, num_splits: int = 1,
                         part_acc=None, part_ml=None, status=None) -> None:
    """``latent_attention`` on tensor cores (bfloat16; see latent_attention_mma_fits).  ``num_splits`` > 1 (single
    tokens only): the key range of a row is cut into pieces that a second kernel merges; part_acc float
    [rows * H * num_splits * R], part_ml float [rows * H * num_splits * 2]."""
    _cuda(qa, cache, sink, out, cu_q, pos0, entry_of_token, block_table, part_acc, part_ml, status)
    T, H, W = qa.shape
    R = out.shape[2]
    assert out.shape == (T, H, R) and cache.shape[1:] == (page_size, W)
    assert out.dtype == cache.dtype == torch.bfloat16
    assert gate is None or (gate.dtype == torch.bfloat16 and gate.stride(1) == 1)   # None: no gate
    assert sink.dtype == torch.float32 and sink.numel() == H and qa.dtype == torch.float32
    if num_splits > 1:
        assert part_acc.dtype == part_ml.dtype == torch.float32 and max_q == 1
        assert part_acc.numel() >= (entry0 + n_entries) * H * num_splits * R
        assert part_ml.numel() >= (entry0 + n_entries) * H * num_splits * 2
    _check(lib().ccb_latent_attention_mma(_p(qa), _p(cache), _p(sink), _p(gate), gate.stride(0) if gate is not None else 0, _p(out), _p(part_acc),
                                          _p(part_ml), num_splits, _p(cu_q), _p(pos0), _p(entry_of_token),
                                          _p(block_table), block_table.stride(0), entry0, n_entries, max_q, H, R,
                                          W - R, page_size, cache.shape[0], int(window), float(scale), _p(status),
                                          _stream()), "latent_attention_mma")
    if num_splits > 1:
        counters.own += 1   # the merge kernel


class RouteRule:
    """How a router turns logits into scores and weights.  ``score``: "softmax" over the experts or "sigmoid" of
    each logit; ``group_top``: a group's score is the sum of this many of its largest choice scores (1 or 2);
    ``renorm``: the chosen scores are divided by their sum (+ 1e-20); ``scale``: the weights' last factor."""

    def __init__(self, score: str = "softmax", group_top: int = 1, renorm: bool = False, scale: float = 1.0):
        if score not in ("softmax", "sigmoid") or group_top not in (1, 2):
            raise Unsupported(f"router rule: score {score!r}, group_top {group_top}")
        self.score, self.group_top, self.renorm, self.scale = score, int(group_top), bool(renorm), float(scale)

    @property
    def args(self):
        return (1 if self.score == "sigmoid" else 0, self.group_top, 1 if self.renorm else 0, self.scale)


_PLAIN_ROUTE = RouteRule()


def moe_route(logits, correction, idx, wts, dense_w, groups: int, keep: int, rule: RouteRule = None,
              E: int = None) -> None:
    """The router's choice per token from float logits [T, E] (more columns may follow in a row): scores by
    ``rule`` (default: softmax, not renormalised), + ``correction`` for the choice, only experts of the ``keep``
    best of ``groups`` groups of neighbours, the top idx.shape[1] of them.  idx int32 [T, top], wts float [T, top]
    (the chosen experts' weights), dense_w (optional) float [T, E]: the same weights as a dense row."""
    _cuda(correction, idx, wts, dense_w)
    T = logits.shape[0]
    if E is None:
        E = dense_w.shape[1] if dense_w is not None else logits.shape[1]
    assert logits.shape[1] >= E
    top = idx.shape[1]
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and idx.dtype == torch.int32
    assert idx.shape == (T, top) and wts.shape == (T, top) and wts.dtype == torch.float32 and idx.is_contiguous()
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == E)
    assert dense_w is None or (dense_w.dtype == torch.float32 and dense_w.shape == (T, E))
    _check(lib().ccb_moe_route(_p(logits), logits.stride(0), _p(correction), _p(idx), _p(wts), _p(dense_w), T, E,
                               int(groups), int(keep), top, *(rule or _PLAIN_ROUTE).args, _stream()), "moe_route")


def moe_dense_glu_act(act, gu, dense_w, E: int, F: int, shared: int, shared_gate=None) -> None:
    """act [T, E F + shared] = silu(gate) * up * weight from the rows ``gu`` [T, 2 (E F + shared)] of ONE product
    over all experts' gate rows and then all their up rows: weight = dense_w[t, e] for expert e's columns (exact
    zeros where it was not chosen); the ``shared`` columns after them get sigmoid(shared_gate[t]) (``shared_gate``
    a float column view [T], or None for 1)."""
    _cuda(dense_w)
    T = act.shape[0]
    W = E * F + shared
    assert act.stride(1) == 1 and gu.stride(1) == 1 and act.shape[1] == W and gu.shape == (T, 2 * W)
    assert act.dtype == gu.dtype and (E == 0 or (dense_w.dtype == torch.float32 and dense_w.shape == (T, E)))
    assert shared_gate is None or (shared_gate.dtype == torch.float32 and shared_gate.shape[0] == T
                                   and shared_gate.dim() == 1)
    _check(lib().ccb_moe_dense_glu_act(_p(act), act.stride(0), _p(gu), gu.stride(0), _p(dense_w), _p(shared_gate),
                                       shared_gate.stride(0) if shared_gate is not None else 0, T, E, F, shared,
                                       _dt(act), _stream()), "moe_dense_glu_act")


def moe_dense_act(act, dense_w, E: int, F: int, shared: int) -> None:
    """In place on the rows of ONE product over all experts' first matrices: act[t, e * F + f] =
    relu(act)^2 * dense_w[t, e]; the ``shared`` columns after the experts get relu(act)^2."""
    _cuda(dense_w)
    T = act.shape[0]
    assert act.stride(1) == 1 and act.shape[1] == E * F + shared and dense_w.dtype == torch.float32
    _check(lib().ccb_moe_dense_act(_p(act), act.stride(0), _p(dense_w), T, E, F, shared, _dt(act), _stream()),
           "moe_dense_act")


def moe_max_tiles(pairs: int, E: int, BM: int) -> int:
    """Tiles of BM rows that the sorted (token, choice) pairs of a step can need at most."""
    return min(pairs, -(-pairs // BM) + E)   # (every tile holds a pair)


def moe_sort(idx, wts, E: int, BM: int, src_row, row_w, pair_pos, tile_e, tile_r0, tile_n) -> None:
    """Sorts the (token, choice) pairs of ``idx`` / ``wts`` [T, top] by expert: pair_pos [T * top] = the sorted
    row of every pair, src_row / row_w = token and weight of every sorted row, tile_* = the tiles of BM rows
    that the experts' rows are cut into (tile_n = 0 for the unused tail of the list)."""
    _cuda(idx, wts, src_row, row_w, pair_pos, tile_e, tile_r0, tile_n)
    T, top = idx.shape
    n_tiles = tile_e.numel()
    assert idx.dtype == torch.int32 and wts.dtype == torch.float32 and wts.shape == (T, top)
    assert src_row.numel() >= T * top and row_w.numel() >= T * top and pair_pos.numel() >= T * top
    assert tile_r0.numel() >= n_tiles and tile_n.numel() >= n_tiles and n_tiles >= moe_max_tiles(T * top, E, BM)
    _check(lib().ccb_moe_sort(_p(idx), _p(wts), T * top, top, E, BM, n_tiles, _p(src_row), _p(row_w), _p(pair_pos),
                              _p(tile_e), _p(tile_r0), _p(tile_n), _stream()), "moe_sort")


MOE_ROUTE_SORT_MAX_TOKENS = 32


def moe_route_sort(logits, correction, idx, wts, groups: int, keep: int, E: int, BM: int, src_row, row_w, pair_pos,
                   tile_e, tile_r0, tile_n, rule: RouteRule = None) -> None:
    """``moe_route`` (without the dense row) and ``moe_sort`` as one kernel, for steps of up to
    MOE_ROUTE_SORT_MAX_TOKENS tokens."""
    _cuda(correction, idx, wts, src_row, row_w, pair_pos, tile_e, tile_r0, tile_n)
    T, top = idx.shape
    n_tiles = tile_e.numel()
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[0] == T and logits.shape[1] >= E
    assert idx.dtype == torch.int32 and idx.is_contiguous() and wts.dtype == torch.float32 and wts.shape == (T, top)
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == E)
    assert src_row.numel() >= T * top and row_w.numel() >= T * top and pair_pos.numel() >= T * top
    assert tile_r0.numel() >= n_tiles and tile_n.numel() >= n_tiles and n_tiles >= moe_max_tiles(T * top, E, BM)
    _check(lib().ccb_moe_route_sort(_p(logits), logits.stride(0), _p(correction), _p(idx), _p(wts), T, E, int(groups),
                                    int(keep), top, BM, n_tiles, _p(src_row), _p(row_w), _p(pair_pos), _p(tile_e),
                                    _p(tile_r0), _p(tile_n), *(rule or _PLAIN_ROUTE).args, _stream()),
           "moe_route_sort")


def moe_grouped(c, a, src_row, w, w_expert_stride: int, row_w, tile_e, tile_r0, tile_n, N: int, K: int, BM: int,
                mode: int) -> None:
    """The product of every tile's rows with its expert's matrix (``w`` [*, ldw] viewed from the first expert's
    first element, expert e at + e * w_expert_stride elements, N rows of K).  mode 0: c[row] = relu(a[src_row[row]]
    W_e^T)^2 * row_w[row] in the compute type; mode 1: c[row] = a[row] W_e^T in float; mode 2: W_e's rows are gate
    and up rows in turn (N of them), c[row] [N / 2] = silu(gate) * up * row_w[row] in the compute type."""
    _cuda(src_row, row_w, tile_e, tile_r0, tile_n)
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1 and a.dtype == w.dtype
    assert c.dtype == (torch.float32 if mode == 1 else a.dtype) and a.shape[1] == K
    assert c.shape[1] == (N // 2 if mode == 2 else N)
    _check(lib().ccb_moe_grouped(_p(a), a.stride(0), _p(src_row), _p(w), w.stride(0), int(w_expert_stride), _p(c),
                                 c.stride(0), _p(row_w), _p(tile_e), _p(tile_r0), _p(tile_n), tile_e.numel(), N, K, BM,
                                 mode, _dt(a), _stream()), "moe_grouped")


MOE_TC_ROWS = 128   # rows of a tile of the tcgen05 grouped product


def moe_gather_rows(out, x, src_row) -> None:
    """out[pos] = x[src_row[pos]]: the tokens of the sorted (token, choice) pairs as contiguous bfloat16 rows."""
    _cuda(out, src_row)
    rows, width = out.shape
    assert x.stride(1) == 1 and x.shape[1] == width and out.dtype == x.dtype == torch.bfloat16
    assert src_row.dtype == torch.int32 and src_row.numel() >= rows
    _check(lib().ccb_moe_gather_rows(_p(out), _p(x), _p(src_row), rows, width, x.stride(0), _stream()),
           "moe_gather_rows")


def moe_grouped_tc(c, a, w, row_w, tile_e, tile_r0, tile_n, N: int, K: int, F: int, mode: int, status=None) -> None:
    """``moe_grouped`` on tcgen05 tensor cores for tiles of MOE_TC_ROWS sorted rows (bfloat16).  ``a`` holds the
    sorted rows themselves.  mode 0: ``w`` = all first matrices stacked [E F, K], c bfloat16 [rows, F] =
    relu(a W_e^T)^2 * row_w;  mode 1: ``w`` = all second matrices side by side [N, E F] (K = F), c float;  mode 2:
    as mode 0 with every expert's F = N rows gate and up rows in turn, c bfloat16 [rows, N / 2] = silu(gate) * up *
    row_w."""
    _cuda(a, w, row_w, tile_e, tile_r0, tile_n, status)
    assert a.dtype == w.dtype == torch.bfloat16 and c.dtype == (torch.float32 if mode == 1 else torch.bfloat16)
    assert a.shape[1] == K and c.shape == (a.shape[0], N // 2 if mode == 2 else N) and c.is_contiguous()
    _check(lib().ccb_moe_grouped_tc(_p(a), a.stride(0), a.shape[0], _p(w), w.stride(0), w.shape[0], w.shape[1], _p(c),
                                    c.stride(0), _p(row_w), _p(tile_e), _p(tile_r0), _p(tile_n), tile_e.numel(), N, K,
                                    F, mode, _p(status), _stream()), "moe_grouped_tc")


def moe_combine(out, rows, pair_pos, shared, top: int) -> None:
    """out[t] = (shared[t]) + sum over the token's choices k of rows[pair_pos[t * top + k]] (float sums in the
    order of the choices); rows float [pairs, D], out and shared [T, D] in the compute type."""
    _cuda(out, rows, pair_pos, shared)
    T, D = out.shape
    assert rows.dtype == torch.float32 and rows.shape[1] == D and pair_pos.dtype == torch.int32
    assert shared is None or (shared.shape == (T, D) and shared.dtype == out.dtype)
    _check(lib().ccb_moe_combine(_p(out), _p(rows), _p(pair_pos), _p(shared), T, top, D, _dt(out), _stream()),
           "moe_combine")


def scaled_residual(h, delta, ls, y=None, w_next=None, eps_next: float = 0.0) -> None:
    """h += delta * ls (a factor per channel); with ``w_next`` y = RMSNorm(h; w_next), else with ``y`` y = h in
    the storage type.  h, ls, w_next float; delta and y in the storage type."""
    _cuda(h, delta, ls, y, w_next)
    T, D = h.shape
    assert h.dtype == torch.float32 and delta.shape == (T, D) and ls.dtype == torch.float32 and ls.numel() == D
    assert y is None or (y.shape == (T, D) and y.dtype == delta.dtype)
    assert w_next is None or (y is not None and w_next.dtype == torch.float32 and w_next.numel() == D)
    _check(lib().ccb_scaled_residual(_p(y), _p(h), _p(delta), _p(ls), _p(w_next), float(eps_next), T, D, _dt(delta),
                                     _stream()), "scaled_residual")


# ---------------------------------------------------------------------------------------------
def embed_pair(h, rows, table, pair_table, ids, positions, entry_of_token, cu_q, state_slot, prev_token, scale: float,
               buckets: int, mul_prev: int, mul_cur: int, n_entries: int, status=None, pending=None) -> None:
    """h[t, :] = float(table[ids[t], :]) * scale + float(pair_table[row, :]) with row = (mul_prev * previous +
    mul_cur * ids[t]) % buckets, or ``buckets`` at position 0; ``pair_table`` None: the first term alone.  The
    previous token of a portion's first token is ``prev_token[slot]`` (int32 [slots]), which afterwards holds the
    portion's last token.  ``rows`` (optional): the same values in the storage type."""
    _cuda(h, rows, table, pair_table, ids, positions, entry_of_token, cu_q, state_slot, prev_token, status, pending)
    T, D = h.shape
    assert h.dtype == torch.float32 and ids.dtype == torch.int32 and table.shape[1] == D
    assert rows is None or (rows.shape == (T, D) and rows.dtype == table.dtype)
    assert pair_table is None or (pair_table.dtype == table.dtype and pair_table.shape == (buckets + 1, D)
                                  and prev_token is not None and prev_token.dtype == torch.int32)
    _check(lib().ccb_embed_pair(_p(h), _p(rows), _p(table), _p(pair_table), _p(ids), _p(positions), _p(entry_of_token),
                                _p(cu_q), _p(state_slot), _p(prev_token), float(scale), int(buckets), int(mul_prev),
                                int(mul_cur), T, int(n_entries), 0 if prev_token is None else prev_token.numel(), D,
                                table.shape[0], _dt(table), _p(pending), 0 if pending is None else pending.numel(),
                                _p(status), _stream()), "embed_pair")
    if pair_table is not None:
        counters.own += 1   # the kernel that stores each request's last token


def relu_squared(act, x) -> None:
    """act = relu(x)^2, elementwise."""
    _cuda(act, x)
    assert act.shape == x.shape and act.dtype == x.dtype
    _check(lib().ccb_relu_squared(_p(act), _p(x), x.numel(), _dt(x), _stream()), "relu_squared")


def scaled_sum(out, a, b, sa: float, sb: float) -> None:
    """out = sa * a + sb * b, elementwise (float arithmetic)."""
    _cuda(out, a, b)
    assert out.shape == a.shape == b.shape and out.dtype == a.dtype == b.dtype
    _check(lib().ccb_scaled_sum(_p(out), _p(a), _p(b), float(sa), float(sb), a.numel(), _dt(a), _stream()),
           "scaled_sum")


def ssm_prepare(proj, ox: int, odt: int, conv_w, conv_b, taps: int, conv_state, A_log, dt_bias, entry_of_token, cu_q,
                state_slot, xs, bs, cs, dts, decay, H: int, P: int, G: int, N: int, shift_single: bool = False) -> None:
    """The inputs of a selective state space recurrence from the input projection's rows ``proj`` [T, >=]: the
    channels x | B | C (from column ``ox``) pass the convolution ``conv_w`` [taps, channels] (+ ``conv_b``) and silu,
    rows before the step's first one coming from ``conv_state`` [slots, taps - 1, channels]; dt = softplus(proj[:,
    odt + h] + dt_bias[h]), decay = exp(-exp(A_log[h]) dt).  Outputs float: xs [T, H, P], bs and cs [T, G, N], dts
    and decay [T, H].  ``shift_single``: a request that brings one token has its convolution state moved on here
    (then ``conv_state_shift`` is for the others only)."""
    _cuda(conv_w, conv_b, conv_state, A_log, dt_bias, entry_of_token, cu_q, state_slot, xs, bs, cs, dts, decay)
    T = xs.shape[0]
    C = H * P + 2 * G * N
    assert proj.stride(1) == 1 and conv_w.dtype == torch.float32 and conv_w.shape == (taps, C)
    assert conv_state is None or (conv_state.dtype == proj.dtype and tuple(conv_state.shape[1:]) == (max(taps - 1, 1), C))
    assert xs.dtype == bs.dtype == cs.dtype == dts.dtype == decay.dtype == torch.float32
    _check(lib().ccb_ssm_prepare(_p(proj), proj.stride(0), int(ox), int(odt), _p(conv_w), _p(conv_b), int(taps),
                                 _p(conv_state), _p(A_log), _p(dt_bias), _p(entry_of_token), _p(cu_q), _p(state_slot),
                                 _p(xs), _p(bs), _p(cs), _p(dts), _p(decay), T, H, P, G, N, 1 if shift_single else 0,
                                 _dt(proj), _stream()), "ssm_prepare")


def conv_state_shift(rows, taps: int, state, cu_q, state_slot, n_entries: int, entry0: int = 0) -> None:
    """After a convolution over a step's rows: the last taps - 1 of (the request's state rows, then its rows of this
    step) become the state [slots, taps - 1, C], for the entries entry0 .. entry0 + n_entries - 1; ``rows`` [T, C]
    may be a column slice of wider rows."""
    _cuda(state, cu_q, state_slot)
    if taps <= 1:
        return
    C = rows.shape[1]
    assert rows.stride(1) == 1 and state.dtype == rows.dtype and tuple(state.shape[1:]) == (taps - 1, C)
    if n_entries <= 0:
        return
    _check(lib().ccb_conv_state_shift(_p(rows), rows.stride(0), int(taps), C, _p(state), _p(cu_q), _p(state_slot),
                                      int(entry0), int(n_entries), state.shape[0], _dt(rows), _stream()),
           "conv_state_shift")


def ssm_recurrence(cs, bs, xs, decay, dts, state, out, cu_q, state_slot, n_entries: int, G: int, H: int, N: int,
                   P: int) -> None:
    """S <- decay_t S + B_t (dt_t x_t)^T, out_t = S^T C_t per head over each request's tokens of the step, from and
    into ``state`` [slots, H, P, N] (float); cs, bs float [T, G, N], xs and out [T, H, P], decay and dts [T, H]."""
    _cuda(cs, bs, xs, decay, dts, state, out, cu_q, state_slot)
    assert state.dtype == torch.float32 and state.shape[1:] == (H, P, N) and out.dtype == torch.float32
    _check(lib().ccb_ssm_recurrence(_p(cs), _p(bs), _p(xs), _p(decay), _p(dts), _p(state), _p(out), _p(cu_q),
                                    _p(state_slot), n_entries, G, H, N, P, _stream()), "ssm_recurrence")


def ssm_gate_norm(y, o, xs, proj, oz: int, skip, w, H: int, P: int, parts: int, eps: float) -> None:
    """y = RMSNorm in ``parts`` equal slices of ((o + skip[h] * xs) * silu(z)) * w; z = proj[:, oz : oz + H P]."""
    _cuda(y, o, xs, skip, w)
    T = y.shape[0]
    assert proj.stride(1) == 1 and proj.dtype == y.dtype and o.dtype == xs.dtype == torch.float32
    assert skip.dtype == w.dtype == torch.float32 and skip.numel() == H and w.numel() == H * P
    _check(lib().ccb_ssm_gate_norm(_p(y), _p(o), _p(xs), _p(proj), proj.stride(0), int(oz), _p(skip), _p(w), T, H, P,
                                   int(parts), float(eps), _dt(y), _stream()), "ssm_gate_norm")


def attention_talking_fits(nq: int, nkv: int, hd: int) -> bool:
    return bool(lib().ccb_attention_talking_fits(int(nq), int(nkv), int(hd)))


TALKING_KEYS = 32   # keys a block takes at a time


def attention_talking_splits(n_rows: int, window: int) -> int:
    """Into how many pieces the key range of a row is cut: enough blocks for two per SM, at most one piece per 32
    keys of a window, 64 at most.  It depends on the number of rows only, so a step of a given size launches one
    grid."""
    most = min(64, -(-window // TALKING_KEYS) + 1) if window else 64
    return max(1, min(most, split_target_blocks() // max(1, n_rows)))


def attention_talking(q, k_cache, v_cache, out, mix, positions, entry_of_token, block_table, window: int,
                      num_splits: int = 1, part_acc=None, part_ml=None, sink=None, gate=None, status=None) -> None:
    """Attention whose heads' scores are mixed before the softmax: s_h = sum_g mix[h, g] (q_g . k), over the pages of
    each row's request; a query at position p sees p - window + 1 .. p (window 0: every j <= p).  q, out
    [T, nq, hd]; caches [pages, nkv, page_size, hd]; ``mix`` float [nq, nq] (with the score scale in it).  ``sink``
    float [nq], ``gate`` [T, >= nq] logits (storage type): see AttnExtra.  ``num_splits`` > 1: the key range in
    pieces, part_acc float [T * splits * nq * hd], part_ml float [T * splits * nq * 2]."""
    _cuda(q, k_cache, v_cache, out, mix, positions, entry_of_token, block_table, part_acc, part_ml, sink, status)
    T, nq, hd = q.shape
    nkv, page_size = k_cache.shape[1], k_cache.shape[2]
    assert out.shape == q.shape and k_cache.shape == v_cache.shape and k_cache.shape[3] == hd
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype and mix.dtype == torch.float32
    assert mix.shape == (nq, nq) and (sink is None or (sink.dtype == torch.float32 and sink.numel() == nq))
    assert gate is None or (gate.dtype == q.dtype and gate.stride(1) == 1)
    if num_splits > 1:
        assert part_acc.numel() >= T * num_splits * nq * hd and part_ml.numel() >= T * num_splits * nq * 2
    _check(lib().ccb_attention_talking(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(part_acc), _p(part_ml), _p(mix),
                                       _p(positions), _p(entry_of_token), _p(block_table), block_table.stride(0), T, nq,
                                       nkv, hd, page_size, k_cache.shape[0], int(window), int(num_splits), _p(sink),
                                       _p(gate), gate.stride(0) if gate is not None else 0, _dt(q), _p(status),
                                       _stream()), "attention_talking")
    if num_splits > 1:
        counters.own += 1   # the merge kernel


def attention_talking_mma_fits(dtype, nq: int, nkv: int, hd: int) -> bool:
    """Whether the tensor-core form of the talking-heads attention takes these sizes (portions of prompts)."""
    return dtype == torch.bfloat16 and bool(lib().ccb_attention_talking_mma_fits(int(nq), int(nkv), int(hd)))


def attention_talking_mma(q, k_cache, v_cache, out, mix, cu_q, pos0, block_table, entry0: int, n_entries: int,
                          max_q: int, window: int, sink=None, gate=None, status=None) -> None:
    """``attention_talking`` for the step's entries entry0 .. entry0 + n_entries - 1 (none with more than ``max_q``
    tokens) on tensor cores: bfloat16, see attention_talking_mma_fits."""
    _cuda(q, k_cache, v_cache, out, mix, cu_q, pos0, block_table, sink, status)
    T, nq, hd = q.shape
    nkv, page_size = k_cache.shape[1], k_cache.shape[2]
    assert out.shape == q.shape and k_cache.shape == v_cache.shape and k_cache.shape[3] == hd
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16 and mix.dtype == torch.float32
    assert mix.shape == (nq, nq) and (sink is None or (sink.dtype == torch.float32 and sink.numel() == nq))
    assert gate is None or (gate.dtype == q.dtype and gate.stride(1) == 1)
    _check(lib().ccb_attention_talking_mma(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(mix), _p(cu_q), _p(pos0),
                                           _p(block_table), block_table.stride(0), int(entry0), int(n_entries),
                                           int(max_q), nq, nkv, hd, page_size, k_cache.shape[0], int(window), _p(sink),
                                           _p(gate), gate.stride(0) if gate is not None else 0, _p(status), _stream()),
           "attention_talking_mma")


def concat_cast(out, a, b) -> None:
    """out[t, :] = [a[t, :] | b[t, :]] in the storage type; a, b float [T, D]."""
    _cuda(out, a, b)
    T, D = a.shape
    assert a.dtype == b.dtype == torch.float32 and b.shape[1] == D and b.shape[0] >= T and out.shape == (T, 2 * D)
    _check(lib().ccb_concat_cast(_p(out), _p(a), _p(b), T, D, _dt(out), _stream()), "concat_cast")


def add_row(h, row) -> None:
    """h[t, :] += row (float)."""
    _cuda(h, row)
    T, D = h.shape
    assert h.dtype == row.dtype == torch.float32 and row.numel() == D
    _check(lib().ccb_add_row(_p(h), _p(row), T, D, _stream()), "add_row")


def gelu_gate_rows(g, table, off: int, ids, status=None, pending=None) -> None:
    """g[t, j] = gelu_tanh(g[t, j]) * table[ids[t], off + j] in place (g [T, n], rows may be strided)."""
    _cuda(table, ids, status, pending)
    T, n = g.shape
    assert g.stride(1) == 1 and g.dtype == table.dtype and ids.dtype == torch.int32 and ids.numel() >= T
    _check(lib().ccb_gelu_gate_rows(_p(g), g.stride(0), _p(table), table.stride(0), int(off), _p(ids), T, n,
                                    table.shape[0], _p(pending), 0 if pending is None else pending.numel(), _dt(g),
                                    _p(status), _stream()), "gelu_gate_rows")


def gemm_f32_batched(c, a, w) -> None:
    """c[b] = a[b] @ w[b]^T for 3-d views [batch, M, *] in true 32-bit arithmetic; rows and batches may be strided."""
    assert c.dtype == a.dtype == w.dtype == torch.float32
    B, M, K = a.shape
    N = w.shape[1]
    assert w.shape == (B, N, K) and c.shape == (B, M, N) and a.stride(2) == w.stride(2) == c.stride(2) == 1
    _check(lib().ccb_gemm_f32_batched(_p(c), _p(a), _p(w), M, N, K, a.stride(1), w.stride(1), c.stride(1),
                                      a.stride(0), w.stride(0), c.stride(0), B, _stream()), "gemm_f32_batched")


def paged_attention_generic(q, k_cache, v_cache, out, positions, entry_of_token, block_table, n_entries: int,
                            window: int, scale: float, status=None) -> None:
    """Causal attention of q [T, nq, hd] over paged caches [pages, nkv, page, hd].

    Token t belongs to request row entry_of_token[t] of block_table [B, stride]
    and sits at absolute position positions[t]; window <= 0 means all keys.
    """
    _cuda(q, k_cache, v_cache, out, positions, entry_of_token, block_table, status)
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    assert hd2 == hd and out.shape == q.shape and q.dtype == k_cache.dtype == v_cache.dtype == out.dtype
    _check(lib().ccb_paged_attention_generic(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(positions),
                                             _p(entry_of_token), _p(block_table), block_table.stride(0),
                                             n_entries, T, nq, nkv, hd, page_size, num_pages, int(window),
                                             float(scale), _dt(q), _p(status), _stream()),
           "paged_attention_generic")


B200_SM_COUNT = 148
_sm_count = None


def sm_count() -> int:
    """SMs of the current CUDA device, asked once.  Without a device: a B200's number, so that the rules
    that size grids can be tabulated on a CPU."""
    global _sm_count
    if _sm_count is None:
        if not torch.cuda.is_available():
            return B200_SM_COUNT
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def split_target_blocks() -> int:
    """Blocks the split attention kernels aim for: two per SM."""
    return 2 * sm_count()


SPLIT_MAX = 32


def attention_split_heads_per_block(nq: int, nkv: int, hd: int) -> int:
    g = nq // nkv
    return 4 if (g >= 4 and hd <= 128) else (2 if g >= 2 else 1)


def attention_split_plan(n_rows: int, nq: int, nkv: int, hd: int, heads_per_block: int = 0):
    """(num_splits, scratch floats for the accumulators, scratch floats for max and sum).

    The number of splits depends on the number of token rows only, so a step of a given size always
    launches the same grid (and its results do not depend on the lengths in the batch)."""
    gt = heads_per_block or attention_split_heads_per_block(nq, nkv, hd)
    per_split = n_rows * nkv * -(-(nq // nkv) // gt)
    target = split_target_blocks()
    splits = max(1, min(SPLIT_MAX, target // max(1, per_split)))
    return splits, target * gt * hd, target * gt * 2


def attention_split(q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table,
                    n_entries: int, row0: int, n_rows: int, window: int, scale: float, num_splits: int,
                    status=None, chunk: int = 0, sink=None, gate=None) -> None:
    """Attention of the token rows row0 .. row0 + n_rows - 1, each a single query with its own position
    and request; the key range is cut into ``num_splits`` pieces merged afterwards (scratch from
    ``attention_split_plan``; unused with one split).  ``chunk`` > 0: a query sees only the keys of its own run of
    ``chunk`` positions (counted from the sequence's start); ``sink`` float [nq]: one more term exp(sink[h]) in
    every softmax denominator of head h; ``gate`` [T, >= nq] (compute type, a view with unit column stride): head
    h's result times sigmoid(gate[t, h])."""
    _cuda(q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table, status, sink)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == q.shape[1])
    assert gate is None or (gate.dtype == q.dtype and gate.stride(1) == 1 and gate.shape[0] == q.shape[0]
                            and gate.shape[1] >= q.shape[1])
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    assert hd2 == hd and out.shape == q.shape and q.dtype == k_cache.dtype == v_cache.dtype == out.dtype
    assert 0 <= row0 and row0 + n_rows <= T
    if num_splits > 1:
        assert part_acc.dtype == part_ml.dtype == torch.float32
        assert part_acc.numel() >= n_rows * nq * num_splits * hd and part_ml.numel() >= n_rows * nq * num_splits * 2
    _check(lib().ccb_attention_split_ex(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(part_acc), _p(part_ml),
                                        _p(positions), _p(entry_of_token), _p(block_table), block_table.stride(0),
                                        n_entries, row0, n_rows, nq, nkv, hd, page_size, num_pages, int(window),
                                        float(scale), num_splits, int(chunk), _p(sink), _p(gate),
                                        gate.stride(0) if gate is not None else 0, _dt(q), _p(status), _stream()),
           "attention_split")
    if num_splits > 1:
        counters.own += 1  # the merge kernel


DECODE_MMA_HEAD_SIZES = (64, 128)
DECODE_MMA_HEADS_PER_BLOCK = 16


def _attn_extra(q_rows: int, nq: int, dtype, chunk: int, sink, gate):
    """The four arguments ``chunk, sink, gate, gate_stride`` of the attention kernels (see ``attention_split``)."""
    _cuda(sink)   # (the gate's rows are a view into a wider row)
    assert chunk >= 0 and (sink is None or (sink.dtype == torch.float32 and sink.numel() == nq))
    assert gate is None or (gate.is_cuda and gate.dtype == dtype and gate.stride(1) == 1 and gate.shape[0] == q_rows
                            and gate.shape[1] >= nq)
    return int(chunk), _p(sink), _p(gate), gate.stride(0) if gate is not None else 0


def attention_decode_mma(q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table,
                         n_entries: int, row0: int, n_rows: int, window: int, scale: float, num_splits: int,
                         status=None, chunk: int = 0, sink=None, gate=None) -> None:
    """As attention_split, on tensor cores: bfloat16, head size 64 or 128, a block per (row, kv head, split)
    serving the whole group of q heads."""
    _cuda(q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table, status)
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    assert hd2 == hd and out.shape == q.shape
    assert q.dtype == k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16
    assert 0 <= row0 and row0 + n_rows <= T
    if num_splits > 1:
        assert part_acc.dtype == part_ml.dtype == torch.float32
        assert part_acc.numel() >= n_rows * nq * num_splits * hd and part_ml.numel() >= n_rows * nq * num_splits * 2
    _check(lib().ccb_attention_decode_mma(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(part_acc), _p(part_ml),
                                          _p(positions), _p(entry_of_token), _p(block_table),
                                          block_table.stride(0), n_entries, row0, n_rows, nq, nkv, hd, page_size,
                                          num_pages, int(window), float(scale), num_splits,
                                          *_attn_extra(T, nq, q.dtype, chunk, sink, gate), _p(status),
                                          _stream()), "attention_decode_mma")
    if num_splits > 1:
        counters.own += 1  # the merge kernel


def attention_decode_tma_fits(hd: int, page_size: int) -> bool:
    return hd in DECODE_MMA_HEAD_SIZES and 8 <= page_size <= 64 and page_size & (page_size - 1) == 0


def attention_decode_tma(q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table,
                         n_entries: int, row0: int, n_rows: int, window: int, scale: float, num_splits: int,
                         status=None, merge_counters=None, chunk: int = 0, sink=None, gate=None) -> None:
    """As attention_decode_mma, with keys and values loaded page by page through TMA boxes by a producer warp
    (page size a power of two from 8 to 64).

    ``merge_counters`` (int32 zeros, left zero): with them the block that finishes last merges the splits
    of its row and head group; without them (or where they are too few) a second kernel does."""
    _cuda(q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table, status, merge_counters)
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    assert hd2 == hd and out.shape == q.shape
    assert q.dtype == k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16
    assert 0 <= row0 and row0 + n_rows <= T
    if num_splits > 1:
        assert part_acc.dtype == part_ml.dtype == torch.float32
        assert part_acc.numel() >= n_rows * nq * num_splits * hd and part_ml.numel() >= n_rows * nq * num_splits * 2
    if merge_counters is not None:
        groups = nkv * -(-(nq // nkv) // DECODE_MMA_HEADS_PER_BLOCK)
        if num_splits == 1 or merge_counters.numel() < n_rows * groups:
            merge_counters = None
        else:
            assert merge_counters.dtype == torch.int32
    _check(lib().ccb_attention_decode_tma(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(part_acc), _p(part_ml),
                                          _p(positions), _p(entry_of_token), _p(block_table),
                                          block_table.stride(0), n_entries, row0, n_rows, nq, nkv, hd, page_size,
                                          num_pages, int(window), float(scale), num_splits, _p(merge_counters),
                                          *_attn_extra(T, nq, q.dtype, chunk, sink, gate), _p(status), _stream()),
           "attention_decode_tma")
    if num_splits > 1 and merge_counters is None:
        counters.own += 1  # the merge kernel


def attention_prefill_mma(q, k_cache, v_cache, out, cu_q, pos0, block_table, entry0: int, n_entries: int,
                          max_new: int, window: int, scale: float, status=None, chunk: int = 0, sink=None,
                          gate=None) -> None:
    """Causal attention of the new tokens of the step's requests entry0 .. entry0 + n_entries - 1 over their
    pages, on tensor cores (bfloat16, head size 64 or 128).  cu_q [B + 1] gives each request's first token
    row, pos0 [B] the position of that token; max_new is the most new tokens any of them has.  ``chunk``,
    ``sink``, ``gate``: as for ``attention_split``."""
    _cuda(q, k_cache, v_cache, out, cu_q, pos0, block_table, status)
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    assert hd2 == hd and out.shape == q.shape
    assert q.dtype == k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16
    assert entry0 >= 0 and entry0 + n_entries <= block_table.shape[0] and cu_q.numel() >= entry0 + n_entries + 1
    _check(lib().ccb_attention_prefill_mma(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(cu_q), _p(pos0),
                                              _p(block_table), block_table.stride(0), entry0, n_entries, max_new,
                                              nq, nkv, hd, page_size, num_pages, int(window), float(scale),
                                              *_attn_extra(T, nq, q.dtype, chunk, sink, gate), _p(status),
                                              _stream()), "attention_prefill_mma")


def attention_decode_tma_fused(qkv, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token,
                               block_table, n_entries: int, row0: int, n_rows: int, nq: int, window: int,
                               scale: float, num_splits: int, q_norm_w, k_norm_w, eps: float, inv_freq,
                               write_kv: bool = True, status=None, merge_counters=None, bias=None,
                               q_temperature=None, chunk: int = 0, sink=None, gate=None) -> None:
    """attention_decode_tma for rows of ONE new token each, straight from the q|k|v product ``qkv``
    [T, (nq + 2 nkv) * hd] (only the nq query heads when ``write_kv`` is false): the kernel norms and rotates
    the queries itself and, with ``write_kv``, also the row's key, which it writes with the value to their
    page and attends to.  qk_norm_rope_kv_write is not needed for these rows.  ``bias`` and ``q_temperature``
    as for ``qkv_bias_rope_kv_write``; ``chunk``, ``sink``, ``gate`` as for ``attention_split``."""
    _cuda(qkv, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table, status,
          merge_counters, q_norm_w, k_norm_w, inv_freq, bias)
    assert bias is None or (write_kv and bias.dtype == torch.float32
                            and bias.numel() == (nq + 2 * k_cache.shape[1]) * k_cache.shape[3])
    T = qkv.shape[0]
    num_pages, nkv, page_size, hd = k_cache.shape
    assert out.shape == (T, nq, hd) and qkv.stride(1) == 1
    assert qkv.dtype == k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16
    assert all(w is None or (w.dtype == torch.float32 and w.numel() >= n) for w, n in
               ((q_norm_w, hd), (k_norm_w, hd), (inv_freq, hd // 2)))
    assert 0 <= row0 and row0 + n_rows <= T
    if num_splits > 1:
        assert part_acc.dtype == part_ml.dtype == torch.float32
        assert part_acc.numel() >= n_rows * nq * num_splits * hd and part_ml.numel() >= n_rows * nq * num_splits * 2
    if merge_counters is not None:
        groups = nkv * -(-(nq // nkv) // DECODE_MMA_HEADS_PER_BLOCK)
        if num_splits == 1 or merge_counters.numel() < n_rows * groups:
            merge_counters = None
    _check(lib().ccb_attention_decode_tma_fused(
        _p(qkv), qkv.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(part_acc), _p(part_ml), _p(positions),
        _p(entry_of_token), _p(block_table), block_table.stride(0), n_entries, row0, n_rows, nq, nkv, hd, page_size,
        num_pages, int(window), float(scale), num_splits, _p(q_norm_w), _p(k_norm_w), float(eps), _p(inv_freq),
        1 if write_kv else 0, _p(bias), float(q_temperature[0]) if q_temperature else 0.0,
        int(q_temperature[1]) if q_temperature else 0, _p(merge_counters),
        *_attn_extra(T, nq, qkv.dtype, chunk, sink, gate), _p(status), _stream()), "attention_decode_tma_fused")
    if num_splits > 1 and merge_counters is None:
        counters.own += 1  # the merge kernel


def attention_prefill_tc_fits(hd: int, page_size: int) -> bool:
    return hd in (64, 128) and 8 <= page_size <= 128 and page_size & (page_size - 1) == 0


def attention_prefill_tc(q, k_cache, v_cache, out, cu_q, pos0, block_table, entry0: int, n_entries: int,
                         max_new: int, window: int, scale: float, status=None, chunk: int = 0, sink=None,
                         gate=None) -> None:
    """As attention_prefill_mma, with both products on tcgen05 tensor cores and the accumulators in tensor
    memory (128-token query tiles, TMA loads page by page).  Page size a power of two from 8 to 128.  Where the
    groups hold an even number of q heads, two heads of a group share a block and its key and value tiles."""
    _cuda(q, k_cache, v_cache, out, cu_q, pos0, block_table, status)
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    assert hd2 == hd and out.shape == q.shape
    assert q.dtype == k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16
    assert entry0 >= 0 and entry0 + n_entries <= block_table.shape[0] and cu_q.numel() >= entry0 + n_entries + 1
    _check(lib().ccb_attention_prefill_tc(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(cu_q), _p(pos0),
                                          _p(block_table), block_table.stride(0), entry0, n_entries, max_new, T,
                                          nq, nkv, hd, page_size, num_pages, int(window), float(scale),
                                          *_attn_extra(T, nq, q.dtype, chunk, sink, gate), _p(status), _stream()),
           "attention_prefill_tc")


def attention_prefill_tc_single_head(on: bool) -> None:
    """Measurements and tests: with ``on`` attention_prefill_tc always runs one q head per block, also where two
    heads of a kv group would share a block (and its key and value tiles)."""
    fn = lib().ccb_attention_prefill_tc_single_head
    fn.argtypes = [c_int]
    fn.restype = c_int
    fn(1 if on else 0)


def gemm_f32(c, a, w) -> None:
    """c[M, N] = a[M, K] @ w[N, K]^T in true 32-bit arithmetic (row strides may exceed the widths)."""
    assert c.dtype == a.dtype == w.dtype == torch.float32 and c.is_cuda and a.is_cuda and w.is_cuda
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    _check(lib().ccb_gemm_f32(_p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), _stream()),
           "gemm_f32")


SKINNY_MAX_ROWS = 16


def gemm_skinny_fits(M: int, K: int, a, w) -> bool:
    """Whether the few-rows product takes this shape (else the library product does)."""
    return (M <= SKINNY_MAX_ROWS and K % 32 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny_bf16(c, a, w) -> None:
    """c[M, N] (bfloat16 or float) = a[M, K] @ w[N, K]^T for M <= 32, K a multiple of 32 (own kernel)."""
    assert a.dtype == w.dtype == torch.bfloat16 and c.dtype in _DT and c.is_cuda and a.is_cuda and w.is_cuda
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    _check(lib().ccb_gemm_skinny_bf16(_p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0),
                                      _dt(c), _stream()), "gemm_skinny_bf16")


TC_SWAP_MAX_ROWS = 64     # up to here the weights are the 128-row side of the tensor-core tile


def tc_target_blocks() -> int:
    """Blocks a tensor-core product of a few rows aims for: one per SM."""
    return sm_count()



def gemm_tc_fits(K: int, a, w) -> bool:
    return (K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def gemm_tc_splits(M: int, N: int, K: int) -> int:
    """How many slices of K run as separate blocks (decode shapes only): enough blocks for every SM."""
    if M > TC_SWAP_MAX_ROWS:
        return 1
    tiles = -(-N // 128)
    kb = -(-K // 64)
    s = max(1, min(-(-tc_target_blocks() // tiles), kb // 4, 16))
    while s > 1 and (s - 1) * (-(-kb // s)) >= kb:   # every slice must hold a k block
        s -= 1
    return s


def gemm_tc_bf16(c, a, w, splits: int = 1, partial=None, counters=None, status=None) -> None:
    """c[M, N] (bfloat16 or float) = a[M, K] @ w[N, K]^T on tcgen05 tensor cores with TMA loads.

    M <= 64 streams the weights as the 128-row operand and may cut K into ``splits`` slices
    (``partial``: float scratch of splits * M * N, ``counters``: int32 zeros, one per 128 features)."""
    assert a.dtype == w.dtype == torch.bfloat16 and c.dtype in _DT and c.is_cuda and a.is_cuda and w.is_cuda
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    if splits > 1:
        assert partial.dtype == torch.float32 and partial.numel() >= splits * M * N
        assert counters.dtype == torch.int32 and counters.numel() >= -(-N // 128)
    _check(lib().ccb_gemm_tc_bf16(_p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), _dt(c),
                                  splits, _p(partial), _p(counters), _p(status), _stream()), "gemm_tc_bf16")


def gemm_tc_pair_bf16(c, a, w, swiglu: bool = False, status=None) -> None:
    """c[M, N] (bfloat16 or float) = a[M, K] @ w[N, K]^T for many rows on tcgen05 tensor cores, two SMs on every
    256 x 256 tile (cta_group::2: each SM holds half of both operands, which halves what its shared memory has
    to deliver per product), one cluster per pair of SMs walking over the tiles, two accumulators in tensor
    memory so that a tile's epilogue runs under the next tile's products.  With ``swiglu`` w [2F, K] is
    interleaved in blocks of SWIGLU_BLOCK rows (interleave_gate_up) and c[M, F] = silu(a Wg^T) * (a Wu^T)."""
    _cuda(w, status)
    assert a.dtype == w.dtype == torch.bfloat16 and c.dtype in _DT and c.is_cuda and a.is_cuda
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N // 2 if swiglu else N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    _check(lib().ccb_gemm_tc_pair_bf16(_p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), _dt(c),
                                       1 if swiglu else 0, sm_count(), _p(status), _stream()), "gemm_tc_pair_bf16")


PAIR_SWIGLU_MIN_ROWS = 1024   # from here on gate|up with the activation fused beats the library product + silu_mul


FEWROWS_MAX_ROWS = 16
FEWROWS_MIN_K = 2048      # below, the register-streaming kernel starts up faster


def gemm_fewrows_fits(M: int, K: int, a, w) -> bool:
    return (M <= FEWROWS_MAX_ROWS and K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_fewrows_bf16(c, a, w, swiglu: bool = False, status=None) -> None:
    """c[M, N] (bfloat16 or float) = a[M, K] @ w[N, K]^T for M <= 16: blocks of 16 features over the whole K
    range, weights and tokens through a TMA ring, mma.sync; with ``swiglu`` w [2F, K] is interleaved in blocks
    of SWIGLU_BLOCK rows (interleave_gate_up) and c[M, F] = silu(a Wg^T) * (a Wu^T)."""
    _cuda(w, status)
    assert a.dtype == w.dtype == torch.bfloat16 and c.dtype in _DT and c.is_cuda and a.is_cuda
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N // 2 if swiglu else N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    _check(lib().ccb_gemm_fewrows_bf16(_p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), _dt(c),
                                       1 if swiglu else 0, _p(status), _stream()), "gemm_fewrows_bf16")


def gemm_fewrows_relu2_bf16(c, a, w, status=None) -> None:
    """c[M, N] = relu(a[M, K] @ w[N, K]^T)^2 for M <= 16: ``gemm_fewrows_bf16`` with the activation as its epilogue."""
    _cuda(w, status)
    assert a.dtype == w.dtype == torch.bfloat16 and c.dtype in _DT and c.is_cuda and a.is_cuda
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    _check(lib().ccb_gemm_fewrows_relu2_bf16(_p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0),
                                             _dt(c), _p(status), _stream()), "gemm_fewrows_relu2_bf16")


def gemm_fewrows_blocks(N: int) -> int:
    """Partial sums per token that gemm_fewrows_norm_bf16 writes when it adds into a residual stream of width N."""
    return int(lib().ccb_gemm_fewrows_blocks(int(N)))


def gemm_fewrows_norm_bf16(c, a, w, swiglu: bool = False, scale=None, into=None, status=None) -> None:
    """gemm_fewrows_bf16 with the halves of an RMSNorm that has no kernel of its own in its epilogue.

    ``scale = (ssq, parts, dim, eps)``: the rows of ``a`` still lack the factor of their norm; token t of the
    result is multiplied by 1 / sqrt(sum_p ssq[t, p] / dim + eps) (before the activation, with ``swiglu``).
    ``into = (h, norm_w, ssq_out)``: h [M, N] (float) += the result; c = bfloat16(h * norm_w); ssq_out
    [16, gemm_fewrows_blocks(N)] gets each block's sum of h^2 per token: what the next product needs as ``scale``."""
    _cuda(w, status)
    assert a.dtype == w.dtype == torch.bfloat16 and c.dtype in _DT and c.is_cuda and a.is_cuda
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N // 2 if swiglu else N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    ssq, parts, dim, eps = scale if scale is not None else (None, 0, 0.0, 0.0)
    h, norm_w, ssq_out = into if into is not None else (None, None, None)
    if ssq is not None:
        assert ssq.dtype == torch.float32 and ssq.is_contiguous() and ssq.numel() >= parts * 16
    if h is not None:
        assert not swiglu and c.dtype == torch.bfloat16 and h.dtype == torch.float32 and h.shape == (M, N)
        assert h.stride(1) == 1 and norm_w.dtype == torch.float32 and norm_w.numel() == N and norm_w.is_contiguous()
        assert ssq_out.dtype == torch.float32 and ssq_out.is_contiguous() and ssq_out.numel() >= gemm_fewrows_blocks(N) * 16
    _check(lib().ccb_gemm_fewrows_norm_bf16(
        _p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), _dt(c), 1 if swiglu else 0,
        _p(ssq), int(parts), float(dim), float(eps), _p(h), h.stride(0) if h is not None else 0, _p(norm_w),
        _p(ssq_out), _p(status), _stream()), "gemm_fewrows_norm_bf16")


def few_rows_product_kernel(M: int, N: int, K: int, sm_count: int, fits_tc: bool, fits_fewrows: bool,
                            fits_skinny: bool) -> str:
    """Which kernel takes out[M, N] = x[M, K] @ w[N, K]^T in bfloat16: "tc", "tc_split", "fewrows", "skinny" or
    "library".  Measured on B200 (graph-timed, weights larger than L2): with up to 16 tokens the tcgen05 kernel
    wins where one block per 128 features fills the machine (gate|up, the vocabulary), the TMA-ring kernel
    with blocks of 16 features on everything smaller from K = 2048 on (q|k|v, o, down).  (For one or two
    tokens it used to have those only where its blocks fit two per SM; since it carries the sum into the
    residual stream and the norm after it in its epilogues, it wins there too: a step of one token at the
    8B / 14B / 32B layer shapes 2.3 / 5.2 / 3.1 % faster.)  What it does not fit goes to the register-streaming
    kernel (short K) or the tcgen05 kernel with K cut into slices (K >= 8192: inside a step the
    register-streaming kernel was 40 us a layer slower there than alone).  More tokens go to the library."""
    if M > SKINNY_MAX_ROWS:
        return "library"
    if fits_tc and -(-N // 128) >= sm_count:
        return "tc"
    if K >= FEWROWS_MIN_K and fits_fewrows:
        return "fewrows"
    if fits_skinny and not (fits_tc and K >= 8192):
        return "skinny"
    if fits_tc:
        return "tc_split"
    return "library"


class CublasHandle:
    """One cuBLAS handle with a caller-owned workspace (no allocation inside a step)."""

    def __init__(self, device, workspace_bytes: int = 64 << 20):
        self._h = c_void_p()
        with torch.cuda.device(device):
            _check(lib().ccb_cublas_create(ctypes.byref(self._h)), "cublas_create")
            self.workspace = torch.empty(workspace_bytes, dtype=torch.uint8, device=device)
            _check(lib().ccb_cublas_set_workspace(self._h, self.workspace.data_ptr(), workspace_bytes),
                   "cublas_set_workspace")

    def gemm_bf16(self, c, a, w) -> None:
        """c[M, N] (bfloat16 or float) = a[M, K] @ w[N, K]^T, bfloat16 operands, float accumulation."""
        assert a.dtype == w.dtype == torch.bfloat16 and c.dtype in _DT
        M, K = a.shape
        N = w.shape[0]
        assert w.shape[1] == K and c.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
        _check(lib().ccb_gemm_bf16(self._h, _p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0),
                                   _dt(c), _stream()), "gemm_bf16")

    def gemm_bf16_batched(self, c, a, w) -> None:
        """c[b] = a[b] @ w[b]^T for 3-d views [batch, M, *]: bfloat16 operands, float accumulation, c bfloat16 or
        float; rows and batches may be strided."""
        assert a.dtype == w.dtype == torch.bfloat16 and c.dtype in _DT
        B, M, K = a.shape
        N = w.shape[1]
        assert w.shape == (B, N, K) and c.shape == (B, M, N) and a.stride(2) == w.stride(2) == c.stride(2) == 1
        _check(lib().ccb_gemm_bf16_batched(self._h, _p(c), _p(a), _p(w), M, N, K, a.stride(1), w.stride(1),
                                           c.stride(1), a.stride(0), w.stride(0), c.stride(0), B, _dt(c), _stream()),
               "gemm_bf16")

    def close(self):
        if self._h:
            lib().ccb_cublas_destroy(self._h)
            self._h = c_void_p()


def sample_rows(logits, tokens, temperature=None, seed=None, out_index=None, slot_of_row=None, by_slot=None,
                top_k=None, top_p=None) -> None:
    """tokens[r] = greedy or temperature draw of logits[r, :] (float), per-row parameters.

    temperature float [R] (<= 0 greedy), seed uint32-valued int32/int64 [R] taken
    as 32 bits, out_index int32 [R].  temperature None = greedy for all rows.
    top_k int32 [R] (0 = off) and top_p float [R] (>= 1 = off) restrict a temperature draw to the k largest
    logits and, within those, to the most probable tokens that hold a share p of the probability.
    With ``slot_of_row`` (int32 [R]) the token of row r is also stored in by_slot[slot_of_row[r]]
    (rows with a slot outside by_slot are skipped).
    """
    _cuda(tokens, temperature, seed, out_index, slot_of_row, by_slot, top_k, top_p)
    assert slot_of_row is None or (slot_of_row.dtype == torch.int32 and by_slot.dtype == torch.int32
                                   and slot_of_row.numel() >= logits.shape[0])
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and tokens.dtype == torch.int32
    assert temperature is None or (temperature.dtype == torch.float32 and seed.dtype == torch.int32
                                   and out_index.dtype == torch.int32)
    assert top_k is None or (top_k.dtype == torch.int32 and top_k.numel() >= R)
    assert top_p is None or (top_p.dtype == torch.float32 and top_p.numel() >= R)
    _check(lib().ccb_sample_rows(_p(logits), logits.stride(0), _p(tokens), _p(temperature), _p(seed),
                                 _p(out_index), _p(top_k), _p(top_p), R, V, _p(slot_of_row), _p(by_slot),
                                 0 if by_slot is None else by_slot.numel(), _stream()), "sample_rows")


def init_random(out: torch.Tensor, seed: int, key: int, std: float, add_one: bool = False) -> None:
    """out (float or bfloat16, contiguous) = std * z (+ 1), z ~ N(0, 1) from the counter-based stream of
    (seed, key); the same bits as ``weights.random_init.normal_host`` (bfloat16: rounded once from float)."""
    _cuda(out)
    _check(lib().ccb_init_random(_p(out), out.numel(), _dt(out), int(seed) & (2 ** 64 - 1), int(key) & (2 ** 64 - 1),
                                 float(std), 1 if add_one else 0, _stream()), "init_random")
