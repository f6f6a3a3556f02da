// Gated delta rule with one decay per head and key channel, as a recurrence over a state per request.
//
// Per head, with S a matrix [key channels, value channels] that starts at zero:
//   S <- diag(g_t) S;  u_t = beta_t (v_t - S^T k_t);  S <- S + k_t u_t^T;  o_t = S^T q_t
// q and k come through a short causal convolution per channel and silu, then are made unit vectors
// per head (q also times dim^-1/2); v comes through its convolution and silu; beta = sigmoid(.),
// g = exp(-exp(A_h) softplus(a + dt_bias)).  Everything after the projections is float.
//
// Four kernels:
//   delta_prepare       a warp per (token, head of q / k / v / decay): convolution + silu, unit norms, beta,
//                       decay -> float rows
//   conv_state_update   the last (taps - 1) projection rows of each request -> its convolution state
//   delta_recurrence    one block per (request, head, 16 value channels): walks the step's tokens of the
//                       request in order; a column of S is independent of the others, so each is held by
//                       8 lanes in registers and 8-lane sums per token give S^T k and S^T q.  The rows of
//                       q, k, g of the next 16 tokens are fetched with cp.async while the current ones are used.
//   gated_head_rmsnorm  o / rms(o) * w * sigmoid(gate) per head -> the compute type
//
// State of a request (slot s): S as [heads, value channels, key channels] floats (a column of S is
// contiguous), and the convolution's last (taps - 1) inputs as [taps - 1, channels] in the compute type.
// Rows whose request has no slot (padding of a replayed step) are skipped.
#include "common.cuh"

using namespace ccb;

namespace {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ---------------------------------------------------------------------------------------------
// proj [T, ld]: columns q (at oq, G*dk), k (at ok, G*dk), v (at ov, H*dv), b (at ob, H); a [T, lda]: H*dk
// decay pre-activations.  conv_w float [taps, C] (tap-major: the channels of a tap side by side) for the
// channels q|k|v in this order (C = 2 G dk + H dv);
// conv_state [slots, taps-1, C].
constexpr int kPrepWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
delta_prepare_kernel(const T* __restrict__ proj, int ld, int oq, int ok, int ov, int ob, const T* __restrict__ a,
                     int lda, const float* __restrict__ conv_w, int taps, const T* __restrict__ conv_state,
                     const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                     const int* __restrict__ entry_of_token, const int* __restrict__ cu_q,
                     const int* __restrict__ state_slot, float* __restrict__ qn, float* __restrict__ kn,
                     float* __restrict__ vv, float* __restrict__ gg, float* __restrict__ bb, int G, int H, int dk,
                     int dv, float q_mult, float unit_eps) {
  ccb::pdl_begin();
  const int t = blockIdx.x;
  const int e = entry_of_token[t];
  if (e < 0) return;
  const int slot = state_slot[e];
  if (slot < 0) return;
  const int lt = t - cu_q[e];  // index of the token within the step's portion of its request
  const int C = 2 * G * dk + H * dv;
  const T* st = conv_state + (size_t)slot * (taps - 1) * C;
  const int lane = threadIdx.x & 31;

  // convolution + silu of channel c (in the order q | k | v), input column `col` of proj
  auto conv = [&](int c, int col) -> float {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {  // tap j multiplies the input (taps - 1 - j) tokens back
      const int back = taps - 1 - j;
      const int li = lt - back;
      float x;
      if (li >= 0) x = to_f32(proj[(size_t)(t - back) * ld + col]);
      else x = to_f32(st[(size_t)(taps - 1 + li) * C + c]);
      acc += conv_w[(size_t)j * C + c] * x;
    }
    return acc * sigmoid_f(acc);
  };

  // units: G query heads, G key heads (unit vectors), H value heads, H decay rows
  const int units = 2 * G + 2 * H;
  const int u = blockIdx.y * kPrepWarps + (threadIdx.x >> 5);   // a warp per unit
  if (u < units) {
    if (u < 2 * G) {
      const bool is_q = u < G;
      const int head = is_q ? u : u - G;
      const int c0 = (is_q ? 0 : G * dk) + head * dk;
      const int col0 = (is_q ? oq : ok) + head * dk;
      float* dst = (is_q ? qn : kn) + ((size_t)t * G + head) * dk;
      float ss = 0.f;
      for (int i = lane; i < dk; i += 32) {
        const float y = conv(c0 + i, col0 + i);
        dst[i] = y;
        ss += y * y;
      }
      ss = warp_sum(ss);
      const float inv = (is_q ? q_mult : 1.0f) / sqrtf(ss + unit_eps);
      for (int i = lane; i < dk; i += 32) dst[i] *= inv;  // each lane rescales what it wrote itself
    } else if (u < 2 * G + H) {
      const int head = u - 2 * G;
      const int c0 = 2 * G * dk + head * dv;
      float* dst = vv + ((size_t)t * H + head) * dv;
      for (int i = lane; i < dv; i += 32) dst[i] = conv(c0 + i, ov + head * dv + i);
      if (lane == 0) bb[(size_t)t * H + head] = sigmoid_f(to_f32(proj[(size_t)t * ld + ob + head]));
    } else {
      const int head = u - 2 * G - H;
      const float rate = expf(A_log[head]);
      float* dst = gg + ((size_t)t * H + head) * dk;
      for (int i = lane; i < dk; i += 32) {
        const float x = to_f32(a[(size_t)t * lda + head * dk + i]) + dt_bias[head * dk + i];
        dst[i] = expf(-rate * softplus_f(x));
      }
    }
  }
}

// The same with four neighbouring channels per lane (16-byte stores, 8- or 16-byte loads): head sizes, column
// offsets, row strides and the channel count are multiples of 4.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
delta_prepare_vec_kernel(const T* __restrict__ proj, int ld, int oq, int ok, int ov, int ob, const T* __restrict__ a,
                         int lda, const float* __restrict__ conv_w, int taps, const T* __restrict__ conv_state,
                         const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                         const int* __restrict__ entry_of_token, const int* __restrict__ cu_q,
                         const int* __restrict__ state_slot, float* __restrict__ qn, float* __restrict__ kn,
                         float* __restrict__ vv, float* __restrict__ gg, float* __restrict__ bb, int G, int H, int dk,
                         int dv, float q_mult, float unit_eps) {
  ccb::pdl_begin();
  const int t = blockIdx.x;
  const int e = entry_of_token[t];
  if (e < 0) return;
  const int slot = state_slot[e];
  if (slot < 0) return;
  const int lt = t - cu_q[e];
  const int C = 2 * G * dk + H * dv;
  const T* st = conv_state + (size_t)slot * (taps - 1) * C;
  const int lane = threadIdx.x & 31;

  // convolution + silu of channels c .. c + 3, input columns col .. col + 3 of proj
  auto conv4 = [&](int c, int col) -> float4 {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;
      const int li = lt - back;
      const float4 x = li >= 0 ? load4(proj + (size_t)(t - back) * ld + col) : load4(st + (size_t)(taps - 1 + li) * C + c);
      const float4 w = load4(conv_w + (size_t)j * C + c);
      acc[0] += w.x * x.x;
      acc[1] += w.y * x.y;
      acc[2] += w.z * x.z;
      acc[3] += w.w * x.w;
    }
    return make_float4(acc[0] * sigmoid_f(acc[0]), acc[1] * sigmoid_f(acc[1]), acc[2] * sigmoid_f(acc[2]),
                       acc[3] * sigmoid_f(acc[3]));
  };

  const int units = 2 * G + 2 * H;
  const int u = blockIdx.y * kPrepWarps + (threadIdx.x >> 5);
  if (u >= units) return;
  if (u < 2 * G) {
    const bool is_q = u < G;
    const int head = is_q ? u : u - G;
    const int c0 = (is_q ? 0 : G * dk) + head * dk;
    const int col0 = (is_q ? oq : ok) + head * dk;
    float* dst = (is_q ? qn : kn) + ((size_t)t * G + head) * dk;
    float4 y[2];   // key sizes up to 256
    float ss = 0.f;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      const int i = 4 * lane + 128 * m;
      if (i < dk) {
        y[m] = conv4(c0 + i, col0 + i);
        ss += y[m].x * y[m].x + y[m].y * y[m].y + y[m].z * y[m].z + y[m].w * y[m].w;
      }
    }
    ss = warp_sum(ss);
    const float inv = (is_q ? q_mult : 1.0f) / sqrtf(ss + unit_eps);
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      const int i = 4 * lane + 128 * m;
      if (i < dk)
        *reinterpret_cast<float4*>(dst + i) = make_float4(y[m].x * inv, y[m].y * inv, y[m].z * inv, y[m].w * inv);
    }
  } else if (u < 2 * G + H) {
    const int head = u - 2 * G;
    const int c0 = 2 * G * dk + head * dv;
    float* dst = vv + ((size_t)t * H + head) * dv;
    for (int i = 4 * lane; i < dv; i += 128) *reinterpret_cast<float4*>(dst + i) = conv4(c0 + i, ov + head * dv + i);
    if (lane == 0) bb[(size_t)t * H + head] = sigmoid_f(to_f32(proj[(size_t)t * ld + ob + head]));
  } else {
    const int head = u - 2 * G - H;
    const float rate = expf(A_log[head]);
    float* dst = gg + ((size_t)t * H + head) * dk;
    for (int i = 4 * lane; i < dk; i += 128) {
      const float4 x = load4(a + (size_t)t * lda + head * dk + i);
      const float4 b = load4(dt_bias + head * dk + i);
      *reinterpret_cast<float4*>(dst + i) =
          make_float4(expf(-rate * softplus_f(x.x + b.x)), expf(-rate * softplus_f(x.y + b.y)),
                      expf(-rate * softplus_f(x.z + b.z)), expf(-rate * softplus_f(x.w + b.w)));
    }
  }
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ proj, int ld, int oq, int ok, int ov,
                                         T* __restrict__ conv_state, int taps, const int* __restrict__ cu_q,
                                         const int* __restrict__ state_slot, int G, int H, int dk, int dv) {
  ccb::pdl_begin();
  const int e = blockIdx.y;
  const int slot = state_slot[e];
  if (slot < 0) return;
  const int C = 2 * G * dk + H * dv;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int col = c < G * dk ? oq + c : (c < 2 * G * dk ? ok + (c - G * dk) : ov + (c - 2 * G * dk));
  const int r0 = cu_q[e], n = cu_q[e + 1] - r0;
  if (n <= 0) return;
  T* st = conv_state + (size_t)slot * (taps - 1) * C;
  // new[i] is the input (taps - 1 - i) tokens before the end; in ascending i an old value is read before
  // its place is written (it sits n >= 1 places further on)
  for (int i = 0; i < taps - 1; ++i) {
    const int li = n - (taps - 1) + i;
    st[(size_t)i * C + c] = li >= 0 ? proj[(size_t)(r0 + li) * ld + col] : st[(size_t)(i + n) * C + c];
  }
}

// ---------------------------------------------------------------------------------------------
constexpr int kLanes = 8;          // lanes that share a column of S
constexpr int kCols = 16;          // columns of S per block
constexpr int kRecThreads = kLanes * kCols;

__device__ __forceinline__ void cp_async4(float* smem, const float* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Rows of a column that lane `lane` holds: in runs of V = min(R, 4) neighbours (one 16-byte access of
// shared memory per run where V = 4), the lanes' runs side by side: row(i) = (i / V) * 8 V + lane V + i % V.
template <int R>
struct Rows {
  static constexpr int V = R < 4 ? R : 4;
  static __device__ __forceinline__ int row(int i, int lane) { return (i / V) * (kLanes * V) + lane * V + (i % V); }
  static __device__ __forceinline__ void load(const float* base, int lane, float* out) {
    if constexpr (V == 4) {
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        const float4 x = *reinterpret_cast<const float4*>(base + j * (kLanes * 4) + lane * 4);
        out[4 * j] = x.x; out[4 * j + 1] = x.y; out[4 * j + 2] = x.z; out[4 * j + 3] = x.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < R; ++i) out[i] = base[row(i, lane)];
    }
  }
};

__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
  for (int o = kLanes / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// R: rows of S per lane (key channels padded to 8 R); C: columns of S per thread, which share the rows of q, k
// and g that the thread has read.  `tch` tokens are staged at a time.
//
// What one token costs is the chain S -> S^T k -> u -> S.  So S^T k and S^T q are both taken from the decayed
// state before the write (o = (gS)^T q + u (k . q), which is the read-out after the write), their sums over
// the lanes run side by side, each sum over a lane's rows is four shorter chains, and the read-out is off the
// chain altogether.
//
// DELTA false: the plain gated recurrence  S <- diag(g_t) S + k_t v_t^T,  o_t = S^T q_t  (gated linear
// attention): u = v, so S^T k and beta are not needed and the chain per token is the decay and one update.
template <int R, int C, bool DELTA>
__global__ void __launch_bounds__(kRecThreads)
delta_recurrence_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vv,
                        const float* __restrict__ gg, const float* __restrict__ bb, float* __restrict__ state,
                        float* __restrict__ out, const int* __restrict__ cu_q, const int* __restrict__ state_slot,
                        int G, int H, int dk, int dv, int tch, int g_dk) {
  ccb::pdl_begin();
  constexpr int DP = R * kLanes;
  constexpr int COLS = kCols * C;   // columns of S per block
  extern __shared__ __align__(16) float smem[];
  const int e = blockIdx.z, head = blockIdx.y;
  const int slot = state_slot[e];
  if (slot < 0) return;
  const int r0 = cu_q[e], n = cu_q[e + 1] - r0;
  if (n <= 0) return;
  const int kvh = head / (H / G);
  const int lane = threadIdx.x & (kLanes - 1);
  const int cl = threadIdx.x / kLanes;
  const int col0 = blockIdx.x * COLS + cl * C;   // this thread's columns: col0 .. col0 + C - 1
  // a stage: q, k, g rows [tch][DP] each, then v [tch][COLS], then beta [tch] (padded to a multiple of 4)
  const int stage_floats = tch * (3 * DP + COLS) + ((tch + 3) & ~3);
  auto sq = [&](int s) { return smem + (size_t)s * stage_floats; };

  // rows past dk never change: q = k = 0, g = 1 there (the loads never touch them)
  for (int s = 0; s < 2; ++s) {
    float* base = sq(s);
    for (int i = threadIdx.x; i < tch * DP; i += kRecThreads) {
      if (i % DP >= dk) {
        base[i] = 0.f;
        base[tch * DP + i] = 0.f;
        base[2 * tch * DP + i] = 1.f;
      }
    }
  }

  auto fetch = [&](int chunk, int s) {
    float* base = sq(s);
    const int t0 = chunk * tch;
    const int cnt = min(tch, n - t0);
    for (int i = threadIdx.x; i < cnt * dk; i += kRecThreads) {
      const int tt = i / dk, r = i - tt * dk;
      const size_t row = (size_t)(r0 + t0 + tt);
      cp_async4(base + tt * DP + r, qn + (row * G + kvh) * dk + r);
      cp_async4(base + tch * DP + tt * DP + r, kn + (row * G + kvh) * dk + r);
      // (g_dk = 1: one decay per head and token, the same for every key channel)
      cp_async4(base + 2 * tch * DP + tt * DP + r, gg + (row * H + head) * g_dk + (g_dk > 1 ? r : 0));
    }
    float* sv = base + 3 * tch * DP;
    for (int i = threadIdx.x; i < cnt * COLS; i += kRecThreads) {
      const int tt = i / COLS, c = i - tt * COLS;
      const int gc = blockIdx.x * COLS + c;
      if (gc < dv) cp_async4(sv + i, vv + ((size_t)(r0 + t0 + tt) * H + head) * dv + gc);
    }
    float* sb = sv + tch * COLS;
    if (DELTA || bb != nullptr)
      for (int i = threadIdx.x; i < cnt; i += kRecThreads) cp_async4(sb + i, bb + (size_t)(r0 + t0 + i) * H + head);
    cp_async_commit();
  };

  float S[C][R];
  float* sp = state + ((size_t)slot * H + head) * dv * dk;
#pragma unroll
  for (int c = 0; c < C; ++c)
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int r = Rows<R>::row(i, lane);
      S[c][i] = (col0 + c < dv && r < dk) ? sp[(size_t)(col0 + c) * dk + r] : 0.f;
    }

  const int chunks = (n + tch - 1) / tch;
  fetch(0, 0);
  for (int ch = 0; ch < chunks; ++ch) {
    cp_async_wait_all();
    __syncthreads();  // chunk ch is in stage ch & 1; everyone is done with stage (ch + 1) & 1
    if (ch + 1 < chunks) fetch(ch + 1, (ch + 1) & 1);
    const float* base = sq(ch & 1);
    const float* sv = base + 3 * tch * DP;
    const float* sb = sv + tch * COLS;
    const int cnt = min(tch, n - ch * tch);
#pragma unroll 2
    for (int tt = 0; tt < cnt; ++tt) {
      float qr[R], kr[R], gr[R];
      Rows<R>::load(base + tt * DP, lane, qr);
      Rows<R>::load(base + tch * DP + tt * DP, lane, kr);
      Rows<R>::load(base + 2 * tch * DP + tt * DP, lane, gr);
      const float beta = (DELTA || bb != nullptr) ? sb[tt] : 1.f;   // (plain form with bb: the write is beta * v)
      constexpr int P = R < 4 ? R : 4;   // partial sums per lane
      float kqp[P];
#pragma unroll
      for (int p = 0; p < P; ++p) kqp[p] = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) kqp[i % P] = fmaf(kr[i], qr[i], kqp[i % P]);
      float kq = kqp[0];
#pragma unroll
      for (int p = 1; p < P; ++p) kq += kqp[p];
      float dkk[C], dqq[C];
#pragma unroll
      for (int c = 0; c < C; ++c) {
        float dkp[P], dqp[P];
#pragma unroll
        for (int p = 0; p < P; ++p) dkp[p] = dqp[p] = 0.f;
#pragma unroll
        for (int i = 0; i < R; ++i) {
          S[c][i] *= gr[i];
          if (DELTA) dkp[i % P] = fmaf(S[c][i], kr[i], dkp[i % P]);
          dqp[i % P] = fmaf(S[c][i], qr[i], dqp[i % P]);
        }
        dkk[c] = dkp[0], dqq[c] = dqp[0];
#pragma unroll
        for (int p = 1; p < P; ++p) dkk[c] += dkp[p], dqq[c] += dqp[p];
      }
      if (DELTA) {
#pragma unroll
        for (int c = 0; c < C; ++c) dkk[c] = lanes_sum(dkk[c]);
      }
      kq = lanes_sum(kq);
#pragma unroll
      for (int c = 0; c < C; ++c) dqq[c] = lanes_sum(dqq[c]);
#pragma unroll
      for (int c = 0; c < C; ++c) {
        const float u = DELTA ? beta * (sv[tt * COLS + cl * C + c] - dkk[c]) : beta * sv[tt * COLS + cl * C + c];
#pragma unroll
        for (int i = 0; i < R; ++i) S[c][i] = fmaf(kr[i], u, S[c][i]);
        if (lane == c % kLanes && col0 + c < dv)
          out[((size_t)(r0 + ch * tch + tt) * H + head) * dv + col0 + c] = fmaf(u, kq, dqq[c]);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < C; ++c)
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int r = Rows<R>::row(i, lane);
      if (col0 + c < dv && r < dk) sp[(size_t)(col0 + c) * dk + r] = S[c][i];
    }
}

// ---------------------------------------------------------------------------------------------
// y[t, h, :] = o[t, h, :] / sqrt(mean(o^2) + eps) * w[:] * sigmoid(gate[t, h, :]); one warp per (t, h).
// SILU: the gate is gate * sigmoid(gate) instead.
template <bool SILU> __device__ __forceinline__ float gate_f(float x) { return SILU ? x * sigmoid_f(x) : sigmoid_f(x); }

template <typename T, bool SILU>
__global__ void gated_head_rmsnorm_kernel(T* __restrict__ y, const float* __restrict__ o, const T* __restrict__ gate,
                                          int ldg, const float* __restrict__ w, int rows, int H, int dv, float eps) {
  ccb::pdl_begin();
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= rows * H) return;
  const int lane = threadIdx.x & 31;
  const int t = unit / H, h = unit - t * H;
  const float* src = o + (size_t)unit * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss += src[i] * src[i];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  const T* gr = gate + (size_t)t * ldg + (size_t)h * dv;
  T* dst = y + (size_t)unit * dv;
  for (int i = lane; i < dv; i += 32) dst[i] = from_f32<T>(src[i] * inv * w[i] * gate_f<SILU>(to_f32(gr[i])));
}

// The same with four neighbouring channels per lane (dv, the gate's row stride and offset multiples of 4).
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 r;
  r.x = *reinterpret_cast<const uint32_t*>(&a);
  r.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = r;
}

template <typename T, bool SILU>
__global__ void gated_head_rmsnorm_vec_kernel(T* __restrict__ y, const float* __restrict__ o,
                                              const T* __restrict__ gate, int ldg, const float* __restrict__ w,
                                              int rows, int H, int dv, float eps) {
  ccb::pdl_begin();
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= rows * H) return;
  const int lane = threadIdx.x & 31;
  const int t = unit / H, h = unit - t * H;
  const float* src = o + (size_t)unit * dv;
  const T* gr = gate + (size_t)t * ldg + (size_t)h * dv;
  constexpr int kMax = 4;   // value sizes up to 512
  float4 x[kMax], g[kMax], ww[kMax];
  float ss = 0.f;
#pragma unroll
  for (int m = 0; m < kMax; ++m) {
    const int i = 4 * lane + 128 * m;
    if (i < dv) {
      x[m] = load4(src + i);
      g[m] = load4(gr + i);
      ww[m] = load4(w + i);
      ss += x[m].x * x[m].x + x[m].y * x[m].y + x[m].z * x[m].z + x[m].w * x[m].w;
    }
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  T* dst = y + (size_t)unit * dv;
#pragma unroll
  for (int m = 0; m < kMax; ++m) {
    const int i = 4 * lane + 128 * m;
    if (i < dv)
      store4<T>(dst + i, make_float4(x[m].x * inv * ww[m].x * gate_f<SILU>(g[m].x), x[m].y * inv * ww[m].y * gate_f<SILU>(g[m].y),
                                     x[m].z * inv * ww[m].z * gate_f<SILU>(g[m].z), x[m].w * inv * ww[m].w * gate_f<SILU>(g[m].w)));
  }
}

}  // namespace

CCB_API int ccb_delta_prepare(const void* proj, int ld, int oq, int ok, int ov, int ob, const void* a, int lda,
                              const float* conv_w, int taps, const void* conv_state, const float* A_log,
                              const float* dt_bias, const int* entry_of_token, const int* cu_q,
                              const int* state_slot, float* qn, float* kn, float* vv, float* gg, float* bb, int T_,
                              int G, int H, int dk, int dv, float q_mult, float unit_eps, int dtype,
                              cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (G <= 0 || H <= 0 || H % G || dk <= 0 || dv <= 0 || taps < 1) return CCB_REFUSE_SIZE;
  const dim3 grid(T_, (2 * G + 2 * H + kPrepWarps - 1) / kPrepWarps);
  const int esz = dtype == CCB_F32 ? 4 : 2;
  const bool vec = (dk % 4 == 0) && (dv % 4 == 0) && dk <= 256 && (ld % 4 == 0) && (lda % 4 == 0) && (oq % 4 == 0) &&
                   (ok % 4 == 0) && (ov % 4 == 0) &&
                   ((reinterpret_cast<uintptr_t>(proj) | reinterpret_cast<uintptr_t>(a) |
                     reinterpret_cast<uintptr_t>(conv_state)) % (4 * esz) == 0) &&
                   ((reinterpret_cast<uintptr_t>(qn) | reinterpret_cast<uintptr_t>(kn) | reinterpret_cast<uintptr_t>(vv) |
                     reinterpret_cast<uintptr_t>(gg) | reinterpret_cast<uintptr_t>(dt_bias) |
                     reinterpret_cast<uintptr_t>(conv_w)) & 15) == 0;
  if (vec && dtype == CCB_F32) {
    ccb_launch(delta_prepare_vec_kernel<float>, grid, dim3(kPrepWarps * 32), 0, stream, (const float*)proj, ld, oq, ok,
               ov, ob, (const float*)a, lda, conv_w, taps, (const float*)conv_state, A_log, dt_bias, entry_of_token,
               cu_q, state_slot, qn, kn, vv, gg, bb, G, H, dk, dv, q_mult, unit_eps);
    return ccb_launch_status();
  }
  if (vec && dtype == CCB_BF16) {
    ccb_launch(delta_prepare_vec_kernel<__nv_bfloat16>, grid, dim3(kPrepWarps * 32), 0, stream,
               (const __nv_bfloat16*)proj, ld, oq, ok, ov, ob, (const __nv_bfloat16*)a, lda, conv_w, taps,
               (const __nv_bfloat16*)conv_state, A_log, dt_bias, entry_of_token, cu_q, state_slot, qn, kn, vv, gg, bb,
               G, H, dk, dv, q_mult, unit_eps);
    return ccb_launch_status();
  }
  if (dtype == CCB_F32)
    ccb_launch(delta_prepare_kernel<float>, grid, dim3(kPrepWarps * 32), 0, stream, (const float*)proj, ld, oq, ok, ov, ob,
               (const float*)a, lda, conv_w, taps, (const float*)conv_state, A_log, dt_bias, entry_of_token, cu_q,
               state_slot, qn, kn, vv, gg, bb, G, H, dk, dv, q_mult, unit_eps);
  else if (dtype == CCB_BF16)
    ccb_launch(delta_prepare_kernel<__nv_bfloat16>, grid, dim3(kPrepWarps * 32), 0, stream, (const __nv_bfloat16*)proj, ld,
               oq, ok, ov, ob, (const __nv_bfloat16*)a, lda, conv_w, taps, (const __nv_bfloat16*)conv_state, A_log,
               dt_bias, entry_of_token, cu_q, state_slot, qn, kn, vv, gg, bb, G, H, dk, dv, q_mult, unit_eps);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

CCB_API int ccb_conv_state_update(const void* proj, int ld, int oq, int ok, int ov, void* conv_state, int taps,
                                  const int* cu_q, const int* state_slot, int n_entries, int G, int H, int dk,
                                  int dv, int dtype, cudaStream_t stream) {
  if (n_entries <= 0 || taps <= 1) return 0;
  const int C = 2 * G * dk + H * dv;
  dim3 grid((C + 255) / 256, n_entries);
  if (dtype == CCB_F32)
    ccb_launch(conv_state_update_kernel<float>, grid, dim3(256), 0, stream, (const float*)proj, ld, oq, ok, ov,
               (float*)conv_state, taps, cu_q, state_slot, G, H, dk, dv);
  else if (dtype == CCB_BF16)
    ccb_launch(conv_state_update_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)proj, ld,
               oq, ok, ov, (__nv_bfloat16*)conv_state, taps, cu_q, state_slot, G, H, dk, dv);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

template <int R, int C, bool DELTA>
static void launch_recurrence(const float* qn, const float* kn, const float* vv, const float* gg, const float* bb,
                              float* state, float* out, const int* cu_q, const int* state_slot, int n_entries, int G,
                              int H, int dk, int dv, cudaStream_t stream, int g_dk) {
  constexpr int DP = R * kLanes, COLS = kCols * C;
  const int tch = DP <= 128 ? 16 : 8;
  const size_t smem = (size_t)2 * (tch * (3 * DP + COLS) + ((tch + 3) & ~3)) * sizeof(float);
  cudaFuncSetAttribute(delta_recurrence_kernel<R, C, DELTA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid((dv + COLS - 1) / COLS, H, n_entries);
  ccb_launch(delta_recurrence_kernel<R, C, DELTA>, grid, dim3(kRecThreads), smem, stream, qn, kn, vv, gg, bb, state, out,
             cu_q, state_slot, G, H, dk, dv, tch, g_dk);
}

template <bool DELTA>
static int pick_recurrence(const float* qn, const float* kn, const float* vv, const float* gg, const float* bb,
                           float* state, float* out, const int* cu_q, const int* state_slot, int n_entries, int G,
                           int H, int dk, int dv, cudaStream_t stream, bool head_decay = false) {
  if (n_entries <= 0) return 0;
  const int g_dk = head_decay ? 1 : dk;
  if (G <= 0 || H <= 0 || H % G || dk <= 0 || dk > 256 || dv <= 0) return CCB_REFUSE_SIZE;
  int R = 1;
  while (R * kLanes < dk) R *= 2;
  // One column per thread.  Two (the rows of q, k, g read once for both) were slower: 1.11 against 0.99 ms
  // for 2,048 tokens of 32 heads of 128 x 128, since the kernel is bound by the latency of what one warp issues
  // per token (with a warp per scheduler an instruction issues every third cycle) and the larger blocks leave
  // fewer warps per SM.  Sixteen lanes a column (twice the warps, one shuffle more per sum) were no faster
  // either (1.03 ms).
#define CCB_REC(RR) \
  launch_recurrence<RR, 1, DELTA>(qn, kn, vv, gg, bb, state, out, cu_q, state_slot, n_entries, G, H, dk, dv, stream, g_dk)
  switch (R) {
    case 1: CCB_REC(1); break;
    case 2: CCB_REC(2); break;
    case 4: CCB_REC(4); break;
    case 8: CCB_REC(8); break;
    case 16: CCB_REC(16); break;
    default: CCB_REC(32); break;
  }
#undef CCB_REC
  return ccb_launch_status();
}

CCB_API int ccb_delta_recurrence(const float* qn, const float* kn, const float* vv, const float* gg,
                                 const float* bb, float* state, float* out, const int* cu_q, const int* state_slot,
                                 int n_entries, int G, int H, int dk, int dv, cudaStream_t stream) {
  return pick_recurrence<true>(qn, kn, vv, gg, bb, state, out, cu_q, state_slot, n_entries, G, H, dk, dv, stream);
}

// The plain gated recurrence (no correction by what the state already holds): S <- diag(g) S + k v^T, o = S^T q.
CCB_API int ccb_gated_linear_recurrence(const float* qn, const float* kn, const float* vv, const float* gg,
                                        float* state, float* out, const int* cu_q, const int* state_slot,
                                        int n_entries, int G, int H, int dk, int dv, cudaStream_t stream) {
  return pick_recurrence<false>(qn, kn, vv, gg, nullptr, state, out, cu_q, state_slot, n_entries, G, H, dk, dv,
                                stream);
}

// The plain recurrence with ONE decay per head and token and a step size on the write (a selective state space
// in its recurrent form):  S <- a_t S + (dt_t v_t-row) ... i.e.  S <- a_t S + k_t (dt_t v_t)^T,  o_t = S^T q_t.
// a and dt float [T, H]; q and k have G groups of dk channels.
CCB_API int ccb_ssm_recurrence(const float* qn, const float* kn, const float* vv, const float* a, const float* dt,
                               float* state, float* out, const int* cu_q, const int* state_slot, int n_entries,
                               int G, int H, int dk, int dv, cudaStream_t stream) {
  if (a == nullptr || dt == nullptr) return CCB_REFUSE_ARG;
  return pick_recurrence<false>(qn, kn, vv, a, dt, state, out, cu_q, state_slot, n_entries, G, H, dk, dv, stream,
                                true);
}

template <typename T, bool SILU>
static void launch_head_norm(bool vec, dim3 grid, void* y, const float* o, const void* gate, int ldg, const float* w,
                             int rows, int H, int dv, float eps, cudaStream_t stream) {
  if (vec)
    ccb_launch(gated_head_rmsnorm_vec_kernel<T, SILU>, grid, dim3(256), 0, stream, (T*)y, o, (const T*)gate, ldg, w,
               rows, H, dv, eps);
  else
    ccb_launch(gated_head_rmsnorm_kernel<T, SILU>, grid, dim3(256), 0, stream, (T*)y, o, (const T*)gate, ldg, w, rows,
               H, dv, eps);
}

// gate_act 0: sigmoid(gate); 1: gate * sigmoid(gate)
CCB_API int ccb_gated_head_rmsnorm(void* y, const float* o, const void* gate, int ldg, const float* w, int rows,
                                   int H, int dv, float eps, int gate_act, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || dv <= 0 || gate_act < 0 || gate_act > 1) return CCB_REFUSE_SIZE;
  const int units = rows * H;
  dim3 grid((units + 7) / 8);
  const int esz = dtype == CCB_F32 ? 4 : 2;
  const bool vec = (dv % 4 == 0) && dv <= 512 && (ldg % 4 == 0) &&
                   ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(w)) & 15) == 0 &&
                   ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(gate)) % (4 * esz)) == 0;
  if (dtype == CCB_F32) {
    if (gate_act) launch_head_norm<float, true>(vec, grid, y, o, gate, ldg, w, rows, H, dv, eps, stream);
    else launch_head_norm<float, false>(vec, grid, y, o, gate, ldg, w, rows, H, dv, eps, stream);
  } else if (dtype == CCB_BF16) {
    if (gate_act) launch_head_norm<__nv_bfloat16, true>(vec, grid, y, o, gate, ldg, w, rows, H, dv, eps, stream);
    else launch_head_norm<__nv_bfloat16, false>(vec, grid, y, o, gate, ldg, w, rows, H, dv, eps, stream);
  } else {
    return CCB_REFUSE_DTYPE;
  }
  return ccb_launch_status();
}
