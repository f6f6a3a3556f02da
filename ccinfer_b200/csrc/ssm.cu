// A selective state space mixer (the recurrent form of state-space duality): what surrounds its recurrence.
//
// The input projection's rows are laid out [z | x | B | C | dt]: a gate z and an input x of `inner` = H P channels,
// G groups of N channels each for B and C, and one step-size logit per head.  x, B and C pass a short causal
// convolution per channel (with bias) followed by silu; the step size is softplus(logit + dt_bias[h]) and the decay
// a = exp(-exp(A_log[h]) * step size).  Head h
// (with group g = h / (H / G)) then runs
//     S <- a_t S + B_t (dt_t x_t)^T        S [N, P], float, kept per request between steps
//     y_t = S^T C_t + D_h x_t
// (the recurrence itself is ccb_ssm_recurrence in delta_rule.cu).  Then y * silu(z) is cut into `parts` equal
// slices of the inner channels, every slice divided by the root of its own mean square (+ eps), and a weight per
// channel is applied.
//
//   ssm_prepare        a thread per (token, channel), or per four channels where sizes and addresses allow: convolution (earlier rows from the step or from the request's
//                      convolution state, which holds its last taps - 1 projected rows), bias, silu; float rows of x,
//                      B, C, and per (token, head) dt and a
//   conv_state_shift   a thread per (request, channel): the last taps - 1 projected rows of each request's portion
//                      become its convolution state (run after ssm_prepare has read the old one).  A request that
//                      brings ONE token is moved on by ssm_prepare itself (`shift_single`): the thread of a channel is
//                      the only one that reads that channel's state, so a decode step needs no second kernel
//   ssm_gate_norm      a block per (token, slice): (o + D x) silu(z), its root mean square, the weight
//
// Everything after the projection is float; the projection's rows and the convolution state are of the storage type.
#include "common.cuh"

using namespace ccb;

namespace {

__device__ __forceinline__ float sigmoid_acc(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_acc(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// proj [T, ld]: the convolved channels (x | B | C, `C` of them) start at column ox, dt at odt.
// conv_w [taps, C] (tap-major), conv_b [C]; conv_state [slots, taps - 1, C].
template <typename T>
__global__ void ssm_prepare_kernel(const T* __restrict__ proj, int ld, int ox, int odt,
                                   const float* __restrict__ conv_w, const float* __restrict__ conv_b, int taps,
                                   const T* conv_state, const float* __restrict__ A_log,
                                   const float* __restrict__ dt_bias, const int* __restrict__ entry_of_token,
                                   const int* __restrict__ cu_q, const int* __restrict__ state_slot,
                                   float* __restrict__ xs, float* __restrict__ bs, float* __restrict__ cs,
                                   float* __restrict__ dts, float* __restrict__ as, int rows, int H, int P, int G, int N,
                                   T* state_rw, int shift_single) {   // (state_rw is conv_state: no __restrict__ on either)
  ccb::pdl_begin();
  const int inner = H * P, gn = G * N;
  const int C = inner + 2 * gn;
  const int per_row = C + H;
  const size_t total = (size_t)rows * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / per_row), c = (int)(i - (size_t)t * per_row);
    const int e = entry_of_token[t];
    if (c >= C) {   // a head's step size and decay
      const int h = c - C;
      float dt = 0.f, a = 1.f;
      if (e >= 0) {
        dt = softplus_acc(to_f32(proj[(size_t)t * ld + odt + h]) + dt_bias[h]);
        a = expf(-expf(A_log[h]) * dt);
      }
      dts[(size_t)t * H + h] = dt;
      as[(size_t)t * H + h] = a;
      continue;
    }
    float v = 0.f;
    if (e >= 0) {
      const int r0 = cu_q[e];
      const int slot = state_slot[e];
      float acc = conv_b ? conv_b[c] : 0.f;
      for (int j = 0; j < taps; ++j) {
        const int src = t - (taps - 1) + j;   // the row this tap reads
        float u;
        if (src >= r0) u = to_f32(proj[(size_t)src * ld + ox + c]);
        else u = slot >= 0 ? to_f32(conv_state[((size_t)slot * (taps - 1) + (src - r0 + taps - 1)) * C + c]) : 0.f;
        acc = fmaf(conv_w[(size_t)j * C + c], u, acc);
      }
      v = acc * sigmoid_acc(acc);
      // a request that brings one token: this thread is the only reader of its channel's state, which it moves on
      if (shift_single && taps > 1 && slot >= 0 && cu_q[e + 1] - r0 == 1) {
        T* st = state_rw + (size_t)slot * (taps - 1) * C + c;
        for (int k = 0; k + 1 < taps - 1; ++k) st[(size_t)k * C] = st[(size_t)(k + 1) * C];
        st[(size_t)(taps - 2) * C] = proj[(size_t)t * ld + ox + c];
      }
    }
    if (c < inner) xs[(size_t)t * inner + c] = v;
    else if (c < inner + gn) bs[(size_t)t * gn + (c - inner)] = v;
    else cs[(size_t)t * gn + (c - inner - gn)] = v;
  }
}


// The same with four neighbouring channels a thread (every width, offset and row stride a multiple of 4, 16-byte
// rows): 8- or 16-byte loads of the rows, 16-byte loads of the weights and stores of the results.
template <typename T> struct In4;
template <> struct In4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
template <> struct In4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 a = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
  }
};

template <typename T>
__global__ void ssm_prepare_vec_kernel(const T* __restrict__ proj, int ld, int ox, int odt,
                                       const float* __restrict__ conv_w, const float* __restrict__ conv_b, int taps,
                                       const T* conv_state, const float* __restrict__ A_log,
                                       const float* __restrict__ dt_bias, const int* __restrict__ entry_of_token,
                                       const int* __restrict__ cu_q, const int* __restrict__ state_slot,
                                       float* __restrict__ xs, float* __restrict__ bs, float* __restrict__ cs,
                                       float* __restrict__ dts, float* __restrict__ as, int rows, int H, int P, int G,
                                       int N, T* state_rw, int shift_single) {   // (state_rw is conv_state: no __restrict__ on either)
  ccb::pdl_begin();
  const int inner = H * P, gn = G * N;
  const int C = inner + 2 * gn;
  const int C4 = C >> 2;
  const int per_row = C4 + H;   // units of a token: groups of four channels, then one per head
  const size_t total = (size_t)rows * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / per_row), u4 = (int)(i - (size_t)t * per_row);
    const int e = entry_of_token[t];
    if (u4 >= C4) {
      const int h = u4 - C4;
      float dt = 0.f, a = 1.f;
      if (e >= 0) {
        dt = softplus_acc(to_f32(proj[(size_t)t * ld + odt + h]) + dt_bias[h]);
        a = expf(-expf(A_log[h]) * dt);
      }
      dts[(size_t)t * H + h] = dt;
      as[(size_t)t * H + h] = a;
      continue;
    }
    const int c = 4 * u4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (e >= 0) {
      const int r0 = cu_q[e];
      const int slot = state_slot[e];
      float4 acc = conv_b ? *reinterpret_cast<const float4*>(conv_b + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < taps; ++j) {
        const int src = t - (taps - 1) + j;
        float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
        if (src >= r0) u = In4<T>::load(proj + (size_t)src * ld + ox + c);
        else if (slot >= 0) u = In4<T>::load(conv_state + ((size_t)slot * (taps - 1) + (src - r0 + taps - 1)) * C + c);
        const float4 wj = *reinterpret_cast<const float4*>(conv_w + (size_t)j * C + c);
        acc.x = fmaf(wj.x, u.x, acc.x);
        acc.y = fmaf(wj.y, u.y, acc.y);
        acc.z = fmaf(wj.z, u.z, acc.z);
        acc.w = fmaf(wj.w, u.w, acc.w);
      }
      v = make_float4(acc.x * sigmoid_acc(acc.x), acc.y * sigmoid_acc(acc.y), acc.z * sigmoid_acc(acc.z),
                      acc.w * sigmoid_acc(acc.w));
      if (shift_single && taps > 1 && slot >= 0 && cu_q[e + 1] - r0 == 1) {   // (as in the kernel above)
        T* st = state_rw + (size_t)slot * (taps - 1) * C + c;
        for (int k = 0; k + 1 < taps - 1; ++k)
          for (int x = 0; x < 4; ++x) st[(size_t)k * C + x] = st[(size_t)(k + 1) * C + x];
        for (int x = 0; x < 4; ++x) st[(size_t)(taps - 2) * C + x] = proj[(size_t)t * ld + ox + c + x];
      }
    }
    float* dst = c < inner ? xs + (size_t)t * inner + c
                           : (c < inner + gn ? bs + (size_t)t * gn + (c - inner) : cs + (size_t)t * gn + (c - inner - gn));
    *reinterpret_cast<float4*>(dst) = v;
  }
}

// state [slots, taps - 1, C] <- the last taps - 1 of (its old rows, then the request's rows of this step).
// A thread owns one (request, channel) and walks the state's rows upwards: row i takes what row i + n held or a row
// of the step, and the rows it still has to read lie above the ones it has written.
template <typename T>
__global__ void conv_state_shift_kernel(const T* __restrict__ rows, int ld, int taps, int C, T* __restrict__ state,
                                        const int* __restrict__ cu_q, const int* __restrict__ state_slot,
                                        int entry0, int n_entries, int n_slots) {
  ccb::pdl_begin();
  const int keep = taps - 1;
  const size_t total = (size_t)n_entries * C;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int e = entry0 + (int)(i / C), c = (int)(i % C);
    const int slot = state_slot[e];
    if (slot < 0 || slot >= n_slots) continue;
    const int r0 = cu_q[e], n = cu_q[e + 1] - r0;
    if (n <= 0) continue;
    T* st = state + (size_t)slot * keep * C + c;
    for (int k = 0; k < keep; ++k) {
      const int src = k + n - keep;   // among the step's rows if >= 0, else the old state's row k + n
      st[(size_t)k * C] = src >= 0 ? rows[(size_t)(r0 + src) * ld + c] : st[(size_t)(k + n) * C];
    }
  }
}

constexpr int kGateThreads = 256;

// y[t, slice] = v / sqrt(mean(v^2) + eps) * w with v = (o + D_h x) * silu(z); o, x float [T, inner], z in proj.
template <typename T>
__global__ void __launch_bounds__(kGateThreads)
ssm_gate_norm_kernel(T* __restrict__ y, const float* __restrict__ o, const float* __restrict__ xs,
                     const T* __restrict__ proj, int ld, int oz, const float* __restrict__ Dskip,
                     const float* __restrict__ w, int P, int inner, int parts, float eps) {
  ccb::pdl_begin();
  __shared__ float red[32];
  const int t = blockIdx.x, part = blockIdx.y;
  const int width = inner / parts;
  const int c0 = part * width;
  const float* orow = o + (size_t)t * inner;
  const float* xrow = xs + (size_t)t * inner;
  const T* zrow = proj + (size_t)t * ld + oz;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += kGateThreads) {
    const int c = c0 + i;
    const float z = to_f32(zrow[c]);
    const float v = fmaf(Dskip[c / P], xrow[c], orow[c]) * (z * sigmoid_acc(z));
    ss += v * v;
  }
  ss = block_sum<kGateThreads>(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += kGateThreads) {
    const int c = c0 + i;
    const float z = to_f32(zrow[c]);
    const float v = fmaf(Dskip[c / P], xrow[c], orow[c]) * (z * sigmoid_acc(z));
    y[(size_t)t * inner + c] = from_f32<T>(v * inv * w[c]);
  }
}

}  // namespace

CCB_API int ccb_ssm_prepare(const void* proj, int ld, int ox, int odt, const float* conv_w, const float* conv_b,
                            int taps, const void* conv_state, const float* A_log, const float* dt_bias,
                            const int* entry_of_token, const int* cu_q, const int* state_slot, float* xs, float* bs,
                            float* cs, float* dts, float* as, int rows, int H, int P, int G, int N, int shift_single,
                            int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || P <= 0 || G <= 0 || N <= 0 || H % G || taps < 1 || taps > 64) return CCB_REFUSE_SIZE;
  if (proj == nullptr || conv_w == nullptr || (taps > 1 && conv_state == nullptr)) return CCB_REFUSE_ARG;
  const int threads = 256;
  const int inner_ = H * P, gn_ = G * N;
  const bool vec = inner_ % 4 == 0 && gn_ % 4 == 0 && ox % 4 == 0 && ld % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(proj) | reinterpret_cast<uintptr_t>(conv_state) |
                     reinterpret_cast<uintptr_t>(conv_w) | reinterpret_cast<uintptr_t>(conv_b) |
                     reinterpret_cast<uintptr_t>(xs) | reinterpret_cast<uintptr_t>(bs) |
                     reinterpret_cast<uintptr_t>(cs)) & 15) == 0;
  if (vec && (dtype == CCB_F32 || dtype == CCB_BF16)) {
    const size_t total4 = (size_t)rows * ((inner_ + 2 * gn_) / 4 + H);
    const size_t want4 = (total4 + threads - 1) / threads;
    const int blocks4 = (int)(want4 < 148 * 32 ? want4 : 148 * 32);
    if (dtype == CCB_F32)
      ccb_launch(ssm_prepare_vec_kernel<float>, blocks4, threads, 0, stream, (const float*)proj, ld, ox, odt, conv_w,
                 conv_b, taps, (const float*)conv_state, A_log, dt_bias, entry_of_token, cu_q, state_slot, xs, bs, cs,
                 dts, as, rows, H, P, G, N, (float*)conv_state, shift_single);
    else
      ccb_launch(ssm_prepare_vec_kernel<__nv_bfloat16>, blocks4, threads, 0, stream, (const __nv_bfloat16*)proj, ld, ox,
                 odt, conv_w, conv_b, taps, (const __nv_bfloat16*)conv_state, A_log, dt_bias, entry_of_token, cu_q,
                 state_slot, xs, bs, cs, dts, as, rows, H, P, G, N, (__nv_bfloat16*)conv_state, shift_single);
    return ccb_launch_status();
  }
  const size_t total = (size_t)rows * (H * P + 2 * G * N + H);
  const size_t want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == CCB_F32)
    ccb_launch(ssm_prepare_kernel<float>, blocks, threads, 0, stream, (const float*)proj, ld, ox, odt, conv_w, conv_b,
               taps, (const float*)conv_state, A_log, dt_bias, entry_of_token, cu_q, state_slot, xs, bs, cs, dts, as,
               rows, H, P, G, N, (float*)conv_state, shift_single);
  else if (dtype == CCB_BF16)
    ccb_launch(ssm_prepare_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (const __nv_bfloat16*)proj, ld, ox, odt,
               conv_w, conv_b, taps, (const __nv_bfloat16*)conv_state, A_log, dt_bias, entry_of_token, cu_q,
               state_slot, xs, bs, cs, dts, as, rows, H, P, G, N, (__nv_bfloat16*)conv_state, shift_single);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

CCB_API int ccb_conv_state_shift(const void* rows, int ld, int taps, int C, void* state, const int* cu_q,
                                 const int* state_slot, int entry0, int n_entries, int n_slots, int dtype,
                                 cudaStream_t stream) {
  if (n_entries <= 0 || taps <= 1) return 0;
  if (C <= 0) return CCB_REFUSE_SIZE;
  const size_t total = (size_t)n_entries * C;
  const int threads = 256;
  const size_t want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == CCB_F32)
    ccb_launch(conv_state_shift_kernel<float>, blocks, threads, 0, stream, (const float*)rows, ld, taps, C,
               (float*)state, cu_q, state_slot, entry0, n_entries, n_slots);
  else if (dtype == CCB_BF16)
    ccb_launch(conv_state_shift_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (const __nv_bfloat16*)rows, ld, taps,
               C, (__nv_bfloat16*)state, cu_q, state_slot, entry0, n_entries, n_slots);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

CCB_API int ccb_ssm_gate_norm(void* y, const float* o, const float* xs, const void* proj, int ld, int oz,
                              const float* Dskip, const float* w, int rows, int H, int P, int parts, float eps,
                              int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int inner = H * P;
  if (H <= 0 || P <= 0 || parts <= 0 || inner % parts) return CCB_REFUSE_SIZE;
  dim3 grid(rows, parts);
  if (dtype == CCB_F32)
    ccb_launch(ssm_gate_norm_kernel<float>, grid, dim3(kGateThreads), 0, stream, (float*)y, o, xs, (const float*)proj,
               ld, oz, Dskip, w, P, inner, parts, eps);
  else if (dtype == CCB_BF16)
    ccb_launch(ssm_gate_norm_kernel<__nv_bfloat16>, grid, dim3(kGateThreads), 0, stream, (__nv_bfloat16*)y, o, xs,
               (const __nv_bfloat16*)proj, ld, oz, Dskip, w, P, inner, parts, eps);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}
