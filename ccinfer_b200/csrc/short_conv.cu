// A short causal convolution over time on the leading channels of a step's projection rows, with the last
// taps - 1 rows of every request kept as its state, and the mixing of a layer's values with those of an earlier
// layer in the same pass.
//
//   y[t, c] = sum_j w[j, c] * u[t - taps + 1 + j, c],   j = 0 .. taps - 1      (w tap-major: a warp's loads of one
//                                                                                tap are consecutive)
//
// where u are the rows of the request in order: the rows this step brings, before them the rows the state
// holds (state[slot, k, c] is the row taps - 1 - k places before the step's first one), zeros before the
// sequence's start (a slot is zeroed when it is given out).  Sums in float, in ascending j.  w null: y = u.
//
// Values: the channels [v_off, v_off + v_heads * v_hd) are value heads of v_hd coordinates of which the first
// v_dim are real.  vmode 1: the results are also left in v_first [tokens, v_heads * v_dim] (compute type);
// vmode 2: y <- (1 - lambda) y + lambda v_first[t], lambda a float on the device.
//
//   conv_rows          a thread per (token, channel); a request that brings ONE token also moves its state on here
//                      (nobody else reads that slot's column in this launch)
//   conv_rows_vec      bfloat16 with every width, stride and offset a multiple of 8: a thread per (token, 8 channels),
//                      16-byte loads and stores; the same sums in the same order
//   conv_state_rows    a thread per (request, channel) for requests that bring several tokens, after conv_rows
#include "common.cuh"

using namespace ccb;

namespace {

constexpr int kConvThreads = 256;
constexpr int kMaxTaps = 16;

template <typename T>
__global__ void __launch_bounds__(kConvThreads)
conv_rows_kernel(const T* __restrict__ in, int in_stride, T* __restrict__ out, int out_stride,
                 const float* __restrict__ w, int taps, int C, T* __restrict__ state,
                 const int* __restrict__ entry_of_token, const int* __restrict__ cu_q,
                 const int* __restrict__ state_slot, int n_entries, int max_slots, int v_off, int v_heads, int v_hd,
                 int v_dim, T* __restrict__ v_first, const float* __restrict__ lambda, int vmode, int* status) {
  ccb::pdl_begin();
  const int t = blockIdx.y;
  const int c = blockIdx.x * kConvThreads + threadIdx.x;
  if (c >= C) return;
  const int b = entry_of_token[t];
  if (b < 0 || b >= n_entries) {   // a padding row: nothing of it is kept
    out[(size_t)t * out_stride + c] = in[(size_t)t * in_stride + c];
    return;
  }
  const int r0 = cu_q[b], n = cu_q[b + 1] - r0, i = t - r0;
  int slot = state != nullptr ? state_slot[b] : -1;   // (one tap, or no convolution: there is no state)
  if (slot >= max_slots) {
    set_status(status, CCB_ST_BAD_SLOT);
    slot = -1;
  }
  const int keep = taps - 1;
  T* st = (slot >= 0 && keep > 0) ? state + (size_t)slot * keep * C + c : nullptr;
  float y;
  if (w == nullptr) {
    y = to_f32(in[(size_t)t * in_stride + c]);
  } else {
    y = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int m = i - keep + j;   // row of the request relative to the step's first one
      float u = 0.f;
      if (m >= 0) u = to_f32(in[(size_t)(r0 + m) * in_stride + c]);
      else if (st != nullptr) u = to_f32(st[(size_t)(keep + m) * C]);
      y = fmaf(w[(size_t)j * C + c], u, y);
    }
    if (n == 1 && st != nullptr) {   // the state moves on by this one row
      for (int k = 0; k + 1 < keep; ++k) st[(size_t)k * C] = st[(size_t)(k + 1) * C];
      st[(size_t)(keep - 1) * C] = in[(size_t)t * in_stride + c];
    }
  }
  if (vmode != 0 && c >= v_off && c < v_off + v_heads * v_hd) {
    const int g = (c - v_off) / v_hd, e = (c - v_off) - g * v_hd;
    if (e < v_dim) {
      const size_t at = (size_t)t * v_heads * v_dim + (size_t)g * v_dim + e;
      if (vmode == 1) {
        v_first[at] = from_f32<T>(y);
      } else {
        const float lam = *lambda;
        y = (1.f - lam) * y + lam * to_f32(v_first[at]);
      }
    }
  }
  out[(size_t)t * out_stride + c] = from_f32<T>(y);
}


// Eight consecutive channels a thread (bfloat16).  The caller has checked that C, the strides, v_off, v_hd, v_dim
// are multiples of 8 and the pointers 16-byte aligned, so that a group of eight never straddles a head's real and
// added coordinates.
__device__ __forceinline__ void unpack8(const uint4 v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(h[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

__global__ void __launch_bounds__(kConvThreads)
conv_rows_vec_kernel(const __nv_bfloat16* __restrict__ in, int in_stride, __nv_bfloat16* __restrict__ out,
                     int out_stride, const float* __restrict__ w, int taps, int C, __nv_bfloat16* __restrict__ state,
                     const int* __restrict__ entry_of_token, const int* __restrict__ cu_q,
                     const int* __restrict__ state_slot, int n_entries, int max_slots, int v_off, int v_heads,
                     int v_hd, int v_dim, __nv_bfloat16* __restrict__ v_first, const float* __restrict__ lambda,
                     int vmode, int* status) {
  ccb::pdl_begin();
  const int t = blockIdx.y;
  const int c = (blockIdx.x * kConvThreads + threadIdx.x) * 8;
  if (c >= C) return;
  const uint4 own = *reinterpret_cast<const uint4*>(in + (size_t)t * in_stride + c);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * out_stride + c);
  const int b = entry_of_token[t];
  if (b < 0 || b >= n_entries) {   // a padding row
    *dst = own;
    return;
  }
  const int r0 = cu_q[b], n = cu_q[b + 1] - r0, i = t - r0;
  int slot = state != nullptr ? state_slot[b] : -1;
  if (slot >= max_slots) {
    set_status(status, CCB_ST_BAD_SLOT);
    slot = -1;
  }
  const int keep = taps - 1;
  __nv_bfloat16* st = (slot >= 0 && keep > 0) ? state + (size_t)slot * keep * C + c : nullptr;
  float y[8];
  if (w == nullptr) {
    unpack8(own, y);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int m = i - keep + j;
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (m == i) raw = own;
      else if (m >= 0) raw = *reinterpret_cast<const uint4*>(in + (size_t)(r0 + m) * in_stride + c);
      else if (st != nullptr) raw = *reinterpret_cast<const uint4*>(st + (size_t)(keep + m) * C);
      float u[8];
      unpack8(raw, u);
      const float4 wa = *reinterpret_cast<const float4*>(w + (size_t)j * C + c);
      const float4 wb = *reinterpret_cast<const float4*>(w + (size_t)j * C + c + 4);
      y[0] = fmaf(wa.x, u[0], y[0]); y[1] = fmaf(wa.y, u[1], y[1]);
      y[2] = fmaf(wa.z, u[2], y[2]); y[3] = fmaf(wa.w, u[3], y[3]);
      y[4] = fmaf(wb.x, u[4], y[4]); y[5] = fmaf(wb.y, u[5], y[5]);
      y[6] = fmaf(wb.z, u[6], y[6]); y[7] = fmaf(wb.w, u[7], y[7]);
    }
    if (n == 1 && st != nullptr) {   // the state moves on by this one row
      for (int k = 0; k + 1 < keep; ++k)
        *reinterpret_cast<uint4*>(st + (size_t)k * C) = *reinterpret_cast<const uint4*>(st + (size_t)(k + 1) * C);
      *reinterpret_cast<uint4*>(st + (size_t)(keep - 1) * C) = own;
    }
  }
  if (vmode != 0 && c >= v_off && c < v_off + v_heads * v_hd) {
    const int g = (c - v_off) / v_hd, e = (c - v_off) - g * v_hd;
    if (e < v_dim) {
      uint4* vf = reinterpret_cast<uint4*>(v_first + (size_t)t * v_heads * v_dim + (size_t)g * v_dim + e);
      if (vmode == 1) {
        *vf = pack8(y);
      } else {
        const float lam = *lambda;
        float f[8];
        unpack8(*vf, f);
#pragma unroll
        for (int q = 0; q < 8; ++q) y[q] = (1.f - lam) * y[q] + lam * f[q];
      }
    }
  }
  *dst = pack8(y);
}

template <typename T>
__global__ void __launch_bounds__(kConvThreads)
conv_state_rows_kernel(const T* __restrict__ in, int in_stride, int taps, int C, T* __restrict__ state,
                       const int* __restrict__ cu_q, const int* __restrict__ state_slot, int entry0, int max_slots) {
  ccb::pdl_begin();
  const int b = entry0 + blockIdx.y;
  const int c = blockIdx.x * kConvThreads + threadIdx.x;
  if (c >= C) return;
  const int r0 = cu_q[b], n = cu_q[b + 1] - r0;
  const int slot = state_slot[b];
  if (n <= 1 || slot < 0 || slot >= max_slots) return;   // single rows were moved on by conv_rows
  const int keep = taps - 1;
  T* st = state + (size_t)slot * keep * C + c;
  for (int k = 0; k < keep; ++k) {   // ascending: an old row is read before its place is written
    const int m = k + n - keep;
    st[(size_t)k * C] = m >= 0 ? in[(size_t)(r0 + m) * in_stride + c] : st[(size_t)(k + n) * C];
  }
}

}  // namespace

CCB_API int ccb_conv_rows(const void* in, int in_stride, void* out, int out_stride, const float* w, int taps, int C,
                          void* state, const int* entry_of_token, const int* cu_q, const int* state_slot,
                          int n_tokens, int n_entries, int max_slots, int v_off, int v_heads, int v_hd, int v_dim,
                          void* v_first, const float* lambda, int vmode, int dtype, int* status,
                          cudaStream_t stream) {
  if (n_tokens <= 0 || C <= 0) return 0;
  if (taps < 1 || taps > kMaxTaps || in_stride < C || out_stride < C || n_tokens > 65535) return CCB_REFUSE_SIZE;
  if (w == nullptr && taps != 1) return CCB_REFUSE_ARG;
  if (taps > 1 && state == nullptr) return CCB_REFUSE_ARG;
  if (vmode < 0 || vmode > 2) return CCB_REFUSE_ARG;
  if (vmode != 0 && (v_first == nullptr || v_hd <= 0 || v_dim <= 0 || v_dim > v_hd || v_off < 0 ||
                     v_off + v_heads * v_hd > C || (vmode == 2 && lambda == nullptr)))
    return CCB_REFUSE_ARG;
  const auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = dtype == CCB_BF16 && C % 8 == 0 && in_stride % 8 == 0 && out_stride % 8 == 0 && al16(in) &&
                   al16(out) && al16(w) && al16(state) &&
                   (vmode == 0 || (v_off % 8 == 0 && v_hd % 8 == 0 && v_dim % 8 == 0 && al16(v_first)));
  if (vec) {
    const dim3 vgrid((C / 8 + kConvThreads - 1) / kConvThreads, n_tokens);
    ccb_launch(conv_rows_vec_kernel, vgrid, dim3(kConvThreads), 0, stream, (const __nv_bfloat16*)in, in_stride,
               (__nv_bfloat16*)out, out_stride, w, taps, C, (__nv_bfloat16*)state, entry_of_token, cu_q, state_slot,
               n_entries, max_slots, v_off, v_heads, v_hd, v_dim, (__nv_bfloat16*)v_first, lambda, vmode, status);
    return ccb_launch_status();
  }
  const dim3 grid((C + kConvThreads - 1) / kConvThreads, n_tokens);
  if (dtype == CCB_F32)
    ccb_launch(conv_rows_kernel<float>, grid, dim3(kConvThreads), 0, stream, (const float*)in, in_stride, (float*)out,
               out_stride, w, taps, C, (float*)state, entry_of_token, cu_q, state_slot, n_entries, max_slots, v_off,
               v_heads, v_hd, v_dim, (float*)v_first, lambda, vmode, status);
  else if (dtype == CCB_BF16)
    ccb_launch(conv_rows_kernel<__nv_bfloat16>, grid, dim3(kConvThreads), 0, stream, (const __nv_bfloat16*)in,
               in_stride, (__nv_bfloat16*)out, out_stride, w, taps, C, (__nv_bfloat16*)state, entry_of_token, cu_q,
               state_slot, n_entries, max_slots, v_off, v_heads, v_hd, v_dim, (__nv_bfloat16*)v_first, lambda, vmode,
               status);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// Entries entry0 .. entry0 + n_entries - 1 (those that bring more than one token; others are skipped).
CCB_API int ccb_conv_state_rows(const void* in, int in_stride, int taps, int C, void* state, const int* cu_q,
                                const int* state_slot, int entry0, int n_entries, int max_slots, int dtype,
                                cudaStream_t stream) {
  if (n_entries <= 0 || C <= 0 || taps <= 1) return 0;
  if (taps > kMaxTaps || in_stride < C || n_entries > 65535 || state == nullptr) return CCB_REFUSE_SIZE;
  const dim3 grid((C + kConvThreads - 1) / kConvThreads, n_entries);
  if (dtype == CCB_F32)
    ccb_launch(conv_state_rows_kernel<float>, grid, dim3(kConvThreads), 0, stream, (const float*)in, in_stride, taps,
               C, (float*)state, cu_q, state_slot, entry0, max_slots);
  else if (dtype == CCB_BF16)
    ccb_launch(conv_state_rows_kernel<__nv_bfloat16>, grid, dim3(kConvThreads), 0, stream, (const __nv_bfloat16*)in,
               in_stride, taps, C, (__nv_bfloat16*)state, cu_q, state_slot, entry0, max_slots);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}
