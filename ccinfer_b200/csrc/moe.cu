// Mixture of experts: the router's choice, and the activation of the experts' first products.
//
// Router (float throughout): s = softmax(z) over all experts, or sigmoid(z) each (RouteRule.score_fn); choice
// scores c = s + correction; the experts form `groups` equal groups of neighbours, a group's score is its largest
// c, or the sum of its two largest (RouteRule.group_top), only experts of the `keep` best groups can be chosen (the
// others count as minus infinity); the `top` largest c are chosen (ties: the lower index); the weight of a
// chosen expert is its s, where RouteRule.renorm says so divided by the chosen ones' sum (+ 1e-20), times
// RouteRule.scale.
//
//   moe_route      a warp per token: idx [T, top] (int32, in the order chosen), wts [T, top], and the same as a
//                  dense row dense_w [T, E] (s where chosen, else 0)
//   moe_dense_act  for the form that runs every expert on every token as ONE product over all experts' rows:
//                  act[t, e * F + f] = relu(u)^2 * dense_w[t, e]; the columns after the experts (a shared expert,
//                  weight 1) get relu(u)^2
#include "common.cuh"
#include <math_constants.h>

using namespace ccb;

namespace {

constexpr int kRouteWarps = 4;

struct RouteRule {
  int score_fn;    // 0: softmax over the experts; 1: sigmoid of each logit
  int group_top;   // a group's score: the sum of this many of its largest choice scores (1 or 2)
  int renorm;      // 1: the chosen scores are divided by their sum (+ 1e-20)
  float scale;     // the weights are multiplied by this last
};

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) v = ov, i = oi;
  }
}

// One token's choice by one warp; s: 2 E + groups floats of shared memory of the warp's own (s[E], c[E], gs[groups]).
__device__ __forceinline__ void route_token(const float* __restrict__ logits, int ldl,
                                            const float* __restrict__ correction, int* __restrict__ idx,
                                            float* __restrict__ wts, float* __restrict__ dense_w, int t, int E,
                                            int groups, int keep, int top, float* s, int lane,
                                            const RouteRule rule) {
  float* c = s + E;
  float* gs = c + E;
  const float* z = logits + (size_t)t * ldl;
  float sum = 1.f;
  if (rule.score_fn == 1) {
    for (int e = lane; e < E; e += 32) s[e] = 1.f / (1.f + expf(-z[e]));
  } else {
    float mx = -CUDART_INF_F;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float v = expf(z[e] - mx);
      s[e] = v;
      sum += v;
    }
    sum = warp_sum(sum);
  }
  for (int e = lane; e < E; e += 32) {
    s[e] = s[e] / sum;
    c[e] = s[e] + (correction ? correction[e] : 0.f);
    if (dense_w) dense_w[(size_t)t * E + e] = 0.f;
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int gsz = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float m = -CUDART_INF_F, m2 = -CUDART_INF_F;   // the largest and the one after it
      for (int j = 0; j < gsz; ++j) {
        const float v = c[g * gsz + j];
        if (v > m) m2 = m, m = v;
        else if (v > m2) m2 = v;
      }
      gs[g] = (rule.group_top >= 2 && gsz >= 2) ? m + m2 : m;
    }
    __syncwarp();
    // the best `keep` groups are marked by +inf in gs, one at a time
    for (int k = 0; k < keep; ++k) {
      float v = -CUDART_INF_F;
      int i = 0x7fffffff;
      for (int g = lane; g < groups; g += 32)
        if (gs[g] != CUDART_INF_F && (gs[g] > v || i == 0x7fffffff)) v = gs[g], i = g;
      warp_argmax(v, i);
      if (lane == 0) gs[i] = CUDART_INF_F;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gs[e / gsz] != CUDART_INF_F) c[e] = -CUDART_INF_F;
    __syncwarp();
  }
  for (int k = 0; k < top; ++k) {
    float v = -CUDART_INF_F;
    int i = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float ce = c[e];
      if (!isnan(ce) && ce != CUDART_INF_F && (ce > v || i == 0x7fffffff)) v = ce, i = e;   // +inf marks a taken one
    }
    warp_argmax(v, i);
    if (lane == 0) {
      idx[(size_t)t * top + k] = i;
      wts[(size_t)t * top + k] = s[i];
      if (dense_w) dense_w[(size_t)t * E + i] = s[i];
      c[i] = CUDART_INF_F;
    }
    __syncwarp();
  }
  if ((rule.renorm || rule.scale != 1.f) && lane == 0) {   // (lane 0 wrote the weights it reads here)
    float f = rule.scale;
    if (rule.renorm) {
      float tot = 0.f;
      for (int k = 0; k < top; ++k) tot += wts[(size_t)t * top + k];
      f = rule.scale / (tot + 1e-20f);
    }
    for (int k = 0; k < top; ++k) {
      const float w = wts[(size_t)t * top + k] * f;
      wts[(size_t)t * top + k] = w;
      if (dense_w) dense_w[(size_t)t * E + idx[(size_t)t * top + k]] = w;
    }
  }
  __syncwarp();
}

// shared memory: a warp's scratch of route_token per warp
__global__ void __launch_bounds__(kRouteWarps * 32)
moe_route_kernel(const float* __restrict__ logits, int ldl, const float* __restrict__ correction,
                 int* __restrict__ idx, float* __restrict__ wts, float* __restrict__ dense_w, int rows, int E,
                 int groups, int keep, int top, RouteRule rule) {
  ccb::pdl_begin();
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + warp;
  if (t >= rows) return;
  route_token(logits, ldl, correction, idx, wts, dense_w, t, E, groups, keep, top,
              smem + (size_t)warp * (2 * E + groups), lane, rule);
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_dense_act_kernel(T* __restrict__ act, int ld, const float* __restrict__ dense_w, int rows, int E, int F,
                     int shared) {
  ccb::pdl_begin();
  const int width = E * F + shared;
  const size_t total = (size_t)rows * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width;
    const int c = (int)(i - t * width);
    T* p = act + t * ld + c;
    float u = fmaxf(to_f32(*p), 0.f);
    u *= u;
    if (c < E * F) {
      const float w = dense_w[t * E + c / F];
      u = w == 0.f ? 0.f : u * w;   // an expert that was not chosen gives exact zeros
    }
    *p = from_f32<T>(u);
  }
}

// Four columns a thread (all widths, the row stride and the base multiples of four columns): the four lie in one
// expert's columns.
template <typename T> struct Row4;
template <> struct Row4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Row4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<const uint32_t*>(&a);
    r.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
  }
};

template <typename T>
__global__ void __launch_bounds__(256)
moe_dense_act_vec_kernel(T* __restrict__ act, int ld, const float* __restrict__ dense_w, int rows, int E, int F,
                         int shared) {
  ccb::pdl_begin();
  const int w4 = (E * F + shared) >> 2;
  const size_t total = (size_t)rows * w4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / w4;
    const int c = (int)(i - t * w4) * 4;
    T* p = act + t * ld + c;
    float4 u = Row4<T>::load(p);
    u.x = fmaxf(u.x, 0.f); u.y = fmaxf(u.y, 0.f); u.z = fmaxf(u.z, 0.f); u.w = fmaxf(u.w, 0.f);
    float w = 1.f;
    if (c < E * F) w = dense_w[t * E + c / F];
    if (w == 0.f) u = make_float4(0.f, 0.f, 0.f, 0.f);   // an expert that was not chosen gives exact zeros
    else u = make_float4(u.x * u.x * w, u.y * u.y * w, u.z * u.z * w, u.w * u.w * w);
    Row4<T>::store(p, u);
  }
}

// The gated form of the same: the product's row holds all gate columns [E F + shared] and then all up columns;
// act[t, c] = silu(gate) * up * weight, weight = dense_w[t, c / F] for an expert's columns (exact zeros where it
// was not chosen) and sigmoid(shared_gate[t * sg_stride]) for the shared expert's (1 where shared_gate is null).
template <typename T>
__global__ void __launch_bounds__(256)
moe_dense_glu_act_kernel(T* __restrict__ act, int lda, const T* __restrict__ gu, int ldg,
                         const float* __restrict__ dense_w, const float* __restrict__ shared_gate, int sg_stride,
                         int rows, int E, int F, int shared) {
  ccb::pdl_begin();
  const int width = E * F + shared;
  const size_t total = (size_t)rows * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width;
    const int c = (int)(i - t * width);
    float w;
    if (c < E * F) w = dense_w[t * E + c / F];
    else w = shared_gate ? 1.f / (1.f + expf(-shared_gate[t * sg_stride])) : 1.f;
    float v = 0.f;
    if (w != 0.f) {
      const float g = to_f32(gu[t * ldg + c]), u = to_f32(gu[t * ldg + width + c]);
      v = g / (1.f + expf(-g)) * u * w;
    }
    act[t * lda + c] = from_f32<T>(v);
  }
}

// The same, bfloat16, eight columns a thread (F, shared, the widths and strides multiples of 8, 16-byte aligned
// rows): the eight lie in one expert's columns and share its weight.  A block row per token, grid-strided.
__global__ void __launch_bounds__(256)
moe_dense_glu_act_vec_kernel(__nv_bfloat16* __restrict__ act, int lda, const __nv_bfloat16* __restrict__ gu, int ldg,
                             const float* __restrict__ dense_w, const float* __restrict__ shared_gate, int sg_stride,
                             int rows, int E, int F, int shared) {
  ccb::pdl_begin();
  const int width = E * F + shared;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= width) return;
  const int e = c < E * F ? c / F : -1;
  for (int t = blockIdx.y; t < rows; t += gridDim.y) {
    float w;
    if (e >= 0) w = dense_w[(size_t)t * E + e];
    else w = shared_gate ? 1.f / (1.f + expf(-shared_gate[(size_t)t * sg_stride])) : 1.f;
    uint4 res = make_uint4(0u, 0u, 0u, 0u);
    if (w != 0.f) {
      const uint4 gv = *reinterpret_cast<const uint4*>(gu + (size_t)t * ldg + c);
      const uint4 uv = *reinterpret_cast<const uint4*>(gu + (size_t)t * ldg + width + c);
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
      const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uv);
      __nv_bfloat162* rh = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 g = __bfloat1622float2(gh[i]), u = __bfloat1622float2(uh[i]);
        rh[i] = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x * w, g.y / (1.f + expf(-g.y)) * u.y * w);
      }
    }
    *reinterpret_cast<uint4*>(act + (size_t)t * lda + c) = res;
  }
}

}  // namespace

CCB_API int ccb_moe_route(const float* logits, int ldl, const float* correction, int* idx, float* wts,
                          float* dense_w, int rows, int E, int groups, int keep, int top, int score_fn,
                          int group_top, int renorm, float scale, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || groups <= 0 || E % groups || keep <= 0 || keep > groups ||
      top > (E / groups) * keep)
    return CCB_REFUSE_SIZE;
  if (score_fn < 0 || score_fn > 1 || group_top < 1 || group_top > 2) return CCB_REFUSE_ARG;
  const RouteRule rule{score_fn, group_top, renorm ? 1 : 0, scale};
  const size_t smem = (size_t)kRouteWarps * (2 * E + groups) * sizeof(float);
  if (smem > 96 * 1024) return CCB_REFUSE_SIZE;
  cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  ccb_launch(moe_route_kernel, dim3((rows + kRouteWarps - 1) / kRouteWarps), dim3(kRouteWarps * 32), smem, stream,
             logits, ldl, correction, idx, wts, dense_w, rows, E, groups, keep, top, rule);
  return ccb_launch_status();
}

CCB_API int ccb_moe_dense_act(void* act, int ld, const float* dense_w, int rows, int E, int F, int shared, int dtype,
                              cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (E < 0 || F <= 0 || shared < 0 || ld < E * F + shared) return CCB_REFUSE_SIZE;
  if (dtype != CCB_F32 && dtype != CCB_BF16) return CCB_REFUSE_DTYPE;
  if ((E == 0 || F % 4 == 0) && shared % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(act) & 15) == 0) {
    const size_t total4 = (size_t)rows * ((E * F + shared) / 4);
    const int blocks4 = (int)((total4 + 255) / 256 < 65535 * 8 ? (total4 + 255) / 256 : 65535 * 8);
    if (dtype == CCB_F32)
      ccb_launch(moe_dense_act_vec_kernel<float>, dim3(blocks4), dim3(256), 0, stream, (float*)act, ld, dense_w, rows,
                 E, F, shared);
    else
      ccb_launch(moe_dense_act_vec_kernel<__nv_bfloat16>, dim3(blocks4), dim3(256), 0, stream, (__nv_bfloat16*)act, ld,
                 dense_w, rows, E, F, shared);
    return ccb_launch_status();
  }
  const size_t total = (size_t)rows * (E * F + shared);
  const int blocks = (int)((total + 255) / 256 < 65535 * 8 ? (total + 255) / 256 : 65535 * 8);
  if (dtype == CCB_F32)
    ccb_launch(moe_dense_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)act, ld, dense_w, rows, E, F,
               shared);
  else if (dtype == CCB_BF16)
    ccb_launch(moe_dense_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)act, ld,
               dense_w, rows, E, F, shared);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// ---------------------------------------------------------------------------------------------
// The sparse form: only the chosen experts run.  The (token, choice) pairs of a step are sorted by expert; the
// rows of an expert are cut into tiles of BM rows and every tile is one block row of a grouped product:
//
//   moe_sort       one block: counts per expert, their prefix sums, the place of every pair among its expert's
//                  rows (pair_pos), the token and weight of every sorted row, and the list of tiles
//   moe_route_sort the router and the sort as ONE block for steps of up to 32 tokens (a warp a token)
//   moe_grouped    C[row, :] = A[src(row), :] W_e^T for the rows of every tile of 16, W_e the tile's expert:
//                  bfloat16 on mma.sync m16n8k16 with float sums.  Both operands go from global memory straight
//                  into the fragments: a thread loads 8 neighbouring k of its rows with ONE 16-byte access and
//                  uses them as two k-pairs of two products.  Which k a fragment's place stands for does not
//                  matter as long as A and B agree, and they do: both load the same way.  (Tiles of 128 rows,
//                  for steps in which an expert gets 8 rows or more on average: moe_tcgen05.cu.)
//                  Epilogues: relu(c)^2 * weight(row) in the compute type (the experts' first product), or
//                  float (the second); moe_combine adds each token's rows up in the order of its choices.
//   The float path has a plain FFMA kernel of the same shape.
#include "mma_common.cuh"

namespace {

constexpr int kSortThreads = 1024;

// idx, wts [pairs] (pairs = tokens * top).  Outputs: src_row [pairs] (token of a sorted row), row_w [pairs],
// pair_pos [pairs] (sorted row of a pair), tile_e / tile_r0 / tile_n [max_tiles].
// The whole block; sm: 4 E + 2 ints of shared memory.
__device__ __forceinline__ void sort_pairs(const int* __restrict__ idx, const float* __restrict__ wts, int pairs,
                                           int top, int E, int BM, int max_tiles, int* __restrict__ src_row,
                                           float* __restrict__ row_w, int* __restrict__ pair_pos,
                                           int* __restrict__ tile_e, int* __restrict__ tile_r0,
                                           int* __restrict__ tile_n, int* sm) {
  const int kSortStride = blockDim.x;
  int* counts = sm;             // [E]
  int* offs = sm + E;           // [E + 1]
  int* tstart = offs + E + 1;   // [E + 1]
  int* cursor = tstart + E + 1; // [E]
  for (int e = threadIdx.x; e < E; e += kSortStride) counts[e] = 0, cursor[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += kSortStride) {
    const int e = idx[p];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, t = 0;
    for (int e = 0; e < E; ++e) {
      offs[e] = o;
      tstart[e] = t;
      o += counts[e];
      t += (counts[e] + BM - 1) / BM;
    }
    offs[E] = o;
    tstart[E] = t;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += kSortStride) {
    const int e = idx[p];
    if (e < 0 || e >= E) { pair_pos[p] = -1; continue; }
    const int pos = offs[e] + atomicAdd(&cursor[e], 1);
    src_row[pos] = p / top;
    row_w[pos] = wts[p];
    pair_pos[p] = pos;
  }
  for (int t = threadIdx.x; t < max_tiles; t += kSortStride) {
    int n = 0, e = 0, r0 = 0;
    if (t < tstart[E]) {
      int lo = 0, hi = E - 1;   // the last expert whose first tile is <= t and that has tiles
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tstart[mid] <= t) lo = mid; else hi = mid - 1;
      }
      e = lo;
      const int j = t - tstart[e];
      r0 = offs[e] + j * BM;
      n = min(BM, counts[e] - j * BM);
    }
    tile_e[t] = e;
    tile_r0[t] = r0;
    tile_n[t] = n;
  }
}

__global__ void __launch_bounds__(kSortThreads)
moe_sort_kernel(const int* __restrict__ idx, const float* __restrict__ wts, int pairs, int top, int E, int BM,
                int max_tiles, int* __restrict__ src_row, float* __restrict__ row_w, int* __restrict__ pair_pos,
                int* __restrict__ tile_e, int* __restrict__ tile_r0, int* __restrict__ tile_n) {
  ccb::pdl_begin();
  extern __shared__ int sm[];
  sort_pairs(idx, wts, pairs, top, E, BM, max_tiles, src_row, row_w, pair_pos, tile_e, tile_r0, tile_n, sm);
}

// Steps of few tokens: the router and the sort in one block, a warp a token (up to 32 tokens).
// Shared memory: the sort's 4 E + 2 ints, then a warp's scratch of route_token per token.
__global__ void __launch_bounds__(kSortThreads)
moe_route_sort_kernel(const float* __restrict__ logits, int ldl, const float* __restrict__ correction,
                      int* __restrict__ idx, float* __restrict__ wts, int rows, int E, int groups, int keep, int top,
                      int BM, int max_tiles, int* __restrict__ src_row, float* __restrict__ row_w,
                      int* __restrict__ pair_pos, int* __restrict__ tile_e, int* __restrict__ tile_r0,
                      int* __restrict__ tile_n, RouteRule rule) {
  ccb::pdl_begin();
  extern __shared__ int sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* scratch = reinterpret_cast<float*>(sm + 4 * E + 2);
  if (warp < rows)
    route_token(logits, ldl, correction, idx, wts, nullptr, warp, E, groups, keep, top,
                scratch + (size_t)warp * (2 * E + groups), lane, rule);
  __threadfence_block();
  __syncthreads();   // the choices are written: the same block sorts them
  sort_pairs(idx, wts, rows * top, top, E, BM, max_tiles, src_row, row_w, pair_pos, tile_e, tile_r0, tile_n, sm);
}

__device__ __forceinline__ uint4 ld16_or_zero(const __nv_bfloat16* p, bool ok) {
  return ok ? *reinterpret_cast<const uint4*>(p) : make_uint4(0u, 0u, 0u, 0u);
}

// MODE 0: C (compute type) = relu(c)^2 * row_w[row];  MODE 1: C (float) = c;  MODE 2: the matrix's rows are
// gate and up rows in turn and C (compute type) [*, N / 2] = silu(gate) * up * row_w[row].
// A [*, lda]: row src_row[r] (MODE 0) or r itself (src_row null).  W_e = W + e * w_expert_stride, rows at ldw.
// Few rows an expert (tiles of 16, a decode step): the product is a stream of the chosen experts' matrices, and
// what counts is bytes in flight.  A block takes 8 columns of a tile; its four warps take a quarter of k each
// (four steps of 32 loaded at once, the next four on their way) and add their parts up through shared memory.
// N / 8 blocks a tile instead of N / 32: every SM holds several, each warp with 2 KB in flight.
template <int MODE>
__global__ void __launch_bounds__(128)
moe_grouped_rows16_kernel(const __nv_bfloat16* __restrict__ A, int lda, const int* __restrict__ src_row,
                          const __nv_bfloat16* __restrict__ W, int ldw, long long w_expert_stride,
                          void* __restrict__ Cout, int ldc, const float* __restrict__ row_w,
                          const int* __restrict__ tile_e, const int* __restrict__ tile_r0,
                          const int* __restrict__ tile_n, int N, int K) {
  ccb::pdl_begin();
  constexpr int DEPTH = 4;
  __shared__ float red[3][32][4];
  const int tile = blockIdx.y;
  const int n_rows = tile_n[tile];
  if (n_rows <= 0) return;
  const int e = tile_e[tile], r0 = tile_r0[tile];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int n_base = blockIdx.x * 8;
  const int col = n_base + gid;
  const bool wok = col < N;
  const __nv_bfloat16* wrow = W + (size_t)e * w_expert_stride + (size_t)(wok ? col : 0) * ldw;
  const __nv_bfloat16* arow[2];
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    int r = hh * 8 + gid;
    if (r >= n_rows) r = n_rows - 1;
    const int g = r0 + r;
    arow[hh] = A + (size_t)(src_row ? src_row[g] : g) * lda;
  }
  // this warp's share of k: whole steps of 32
  const int steps = (K + 31) >> 5, per = (steps + 3) >> 2;
  const int k_begin = warp * per * 32, k_end = min(K, (warp + 1) * per * 32);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  uint4 a[DEPTH][2], b[DEPTH];
  auto load = [&](int k0) {
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      const int k = k0 + 32 * d + 8 * tig;
      const bool ok = k < k_end;
      a[d][0] = ld16_or_zero(arow[0] + k, ok);
      a[d][1] = ld16_or_zero(arow[1] + k, ok);
      b[d] = ld16_or_zero(wrow + k, ok && wok);
    }
  };
  if (k_begin < k_end) load(k_begin);
  for (int k0 = k_begin; k0 < k_end; k0 += 32 * DEPTH) {
    uint4 ca[DEPTH][2], cb[DEPTH];
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) ca[d][0] = a[d][0], ca[d][1] = a[d][1], cb[d] = b[d];
    if (k0 + 32 * DEPTH < k_end) load(k0 + 32 * DEPTH);
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      const uint32_t f0[4] = {ca[d][0].x, ca[d][1].x, ca[d][0].y, ca[d][1].y};
      const uint32_t f1[4] = {ca[d][0].z, ca[d][1].z, ca[d][0].w, ca[d][1].w};
      mma_bf16_16816(acc, f0, cb[d].x, cb[d].y);
      mma_bf16_16816(acc, f1, cb[d].z, cb[d].w);
    }
  }
  if (warp > 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) red[warp - 1][lane][i] = acc[i];
  }
  __syncthreads();
  if (warp > 0) return;
#pragma unroll
  for (int w = 0; w < 3; ++w)   // the quarters of k are added in their order
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] += red[w][lane][i];
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int r = hh * 8 + gid;
    if (r >= n_rows) continue;
    const size_t g = (size_t)(r0 + r);
    const int c0 = n_base + 2 * tig;
    float v0 = acc[hh * 2], v1 = acc[hh * 2 + 1];
    if (MODE == 0) {
      const float wr = row_w[g];
      v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f);
      v0 = v0 * v0 * wr; v1 = v1 * v1 * wr;
      __nv_bfloat16* c = (__nv_bfloat16*)Cout + g * ldc + c0;
      if (c0 < N) c[0] = __float2bfloat16_rn(v0);
      if (c0 + 1 < N) c[1] = __float2bfloat16_rn(v1);
    } else if (MODE == 2) {   // columns (2 f, 2 f + 1) are gate f and up f: one number of the gated activation
      if (c0 + 1 < N)
        ((__nv_bfloat16*)Cout)[g * ldc + (c0 >> 1)] = __float2bfloat16_rn(v0 / (1.f + __expf(-v0)) * v1 * row_w[g]);
    } else {
      float* c = (float*)Cout + g * ldc + c0;
      if (c0 < N) c[0] = v0;
      if (c0 + 1 < N) c[1] = v1;
    }
  }
}

// The float path: a tile of up to 16 rows x 128 columns a block, a column a thread, A staged in shared memory.
template <int MODE>
__global__ void __launch_bounds__(128)
moe_grouped_f32_kernel(const float* __restrict__ A, int lda, const int* __restrict__ src_row,
                       const float* __restrict__ W, int ldw, long long w_expert_stride, float* __restrict__ C, int ldc,
                       const float* __restrict__ row_w, const int* __restrict__ tile_e,
                       const int* __restrict__ tile_r0, const int* __restrict__ tile_n, int N, int K) {
  ccb::pdl_begin();
  constexpr int KC = 32;
  __shared__ float As[16][KC];
  const int tile = blockIdx.x;
  const int n_rows = tile_n[tile];
  if (n_rows <= 0) return;
  const int e = tile_e[tile], r0 = tile_r0[tile];
  const int col = blockIdx.y * 128 + threadIdx.x;
  const float* wr = W + (size_t)e * w_expert_stride + (size_t)(col < N ? col : 0) * ldw;
  float acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.f;
  for (int k0 = 0; k0 < K; k0 += KC) {
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * KC; i += 128) {
      const int r = i / KC, k = k0 + i % KC;
      float v = 0.f;
      if (r < n_rows && k < K) {
        const int g = r0 + r;
        v = A[(size_t)(src_row ? src_row[g] : g) * lda + k];
      }
      As[r][i % KC] = v;
    }
    __syncthreads();
    const int kn = min(KC, K - k0);
    for (int k = 0; k < kn; ++k) {
      const float w = wr[k0 + k];
#pragma unroll
      for (int r = 0; r < 16; ++r) acc[r] = fmaf(As[r][k], w, acc[r]);
    }
  }
  if (MODE == 2) {   // columns (2 f, 2 f + 1) are gate f and up f (N is even: a pair lies in one warp)
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      const float up = __shfl_down_sync(0xffffffffu, acc[r], 1);
      if (r < n_rows && col + 1 < N && !(col & 1))
        C[(size_t)(r0 + r) * ldc + (col >> 1)] = acc[r] / (1.f + expf(-acc[r])) * up * row_w[r0 + r];
    }
    return;
  }
  if (col >= N) return;
  for (int r = 0; r < n_rows; ++r) {
    float v = acc[r];
    if (MODE == 0) {
      v = fmaxf(v, 0.f);
      v = v * v * row_w[r0 + r];
    }
    C[(size_t)(r0 + r) * ldc + col] = v;
  }
}

// out[t, :] = (shared ? shared[t, :] : 0) + sum_k rows[pair_pos[t * top + k], :]   (float sums, fixed order)
template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(T* __restrict__ out, const float* __restrict__ rows, const int* __restrict__ pair_pos,
                   const T* __restrict__ shared, int top, int D, size_t total) {
  ccb::pdl_begin();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / D;
    const int c = (int)(i - t * D);
    float v = 0.f;
    for (int k = 0; k < top; ++k) {
      const int pos = pair_pos[t * top + k];
      if (pos >= 0) v += rows[(size_t)pos * D + c];
    }
    if (shared) v += to_f32(shared[i]);
    out[i] = from_f32<T>(v);
  }
}

// the same, four columns a thread (D a multiple of 4, 16-byte rows)
template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_vec_kernel(T* __restrict__ out, const float* __restrict__ rows, const int* __restrict__ pair_pos,
                       const T* __restrict__ shared, int top, int D, size_t total4) {
  ccb::pdl_begin();
  const int d4 = D >> 2;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / d4;
    const int c = (int)(i - t * d4) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < top; ++k) {
      const int pos = pair_pos[t * top + k];
      if (pos >= 0) {
        const float4 x = *reinterpret_cast<const float4*>(rows + (size_t)pos * D + c);
        v.x += x.x; v.y += x.y; v.z += x.z; v.w += x.w;
      }
    }
    if (shared) {
      const float4 x = Row4<T>::load(shared + t * D + c);
      v.x += x.x; v.y += x.y; v.z += x.z; v.w += x.w;
    }
    Row4<T>::store(out + t * D + c, v);
  }
}

}  // namespace

CCB_API int ccb_moe_sort(const int* idx, const float* wts, int pairs, int top, int E, int BM, int max_tiles,
                         int* src_row, float* row_w, int* pair_pos, int* tile_e, int* tile_r0, int* tile_n,
                         cudaStream_t stream) {
  if (pairs <= 0) return 0;
  // (every tile holds a pair, so there are never more tiles than pairs)
  if (E <= 0 || top <= 0 || BM <= 0 || max_tiles < min(pairs, (pairs + BM - 1) / BM + E)) return CCB_REFUSE_SIZE;
  const size_t smem = (size_t)(4 * E + 2) * sizeof(int);
  if (smem > 96 * 1024) return CCB_REFUSE_SIZE;
  cudaFuncSetAttribute(moe_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  ccb_launch(moe_sort_kernel, dim3(1), dim3(kSortThreads), smem, stream, idx, wts, pairs, top, E, BM, max_tiles,
             src_row, row_w, pair_pos, tile_e, tile_r0, tile_n);
  return ccb_launch_status();
}

// ccb_moe_route and ccb_moe_sort in one kernel, for up to 32 tokens (no dense row of weights).
CCB_API int ccb_moe_route_sort(const float* logits, int ldl, const float* correction, int* idx, float* wts, int rows,
                               int E, int groups, int keep, int top, int BM, int max_tiles, int* src_row, float* row_w,
                               int* pair_pos, int* tile_e, int* tile_r0, int* tile_n, int score_fn, int group_top,
                               int renorm, float scale, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (score_fn < 0 || score_fn > 1 || group_top < 1 || group_top > 2) return CCB_REFUSE_ARG;
  const RouteRule rule{score_fn, group_top, renorm ? 1 : 0, scale};
  if (rows > 32 || E <= 0 || top <= 0 || top > E || groups <= 0 || E % groups || keep <= 0 || keep > groups ||
      top > (E / groups) * keep || BM <= 0 || max_tiles < min(rows * top, (rows * top + BM - 1) / BM + E))
    return CCB_REFUSE_SIZE;
  const size_t smem = (size_t)(4 * E + 2) * sizeof(int) + (size_t)rows * (2 * E + groups) * sizeof(float);
  if (smem > 96 * 1024) return CCB_REFUSE_SIZE;
  cudaFuncSetAttribute(moe_route_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  ccb_launch(moe_route_sort_kernel, dim3(1), dim3(kSortThreads), smem, stream, logits, ldl, correction, idx, wts, rows,
             E, groups, keep, top, BM, max_tiles, src_row, row_w, pair_pos, tile_e, tile_r0, tile_n, rule);
  return ccb_launch_status();
}

// mode 0: C (the compute type) [sorted rows, N] = relu(A[src_row] W_e^T)^2 * row_w;  mode 1: C (float) = A W_e^T
// with A's rows the sorted rows themselves;  mode 2: W_e's N rows are gate and up rows in turn, C (the compute
// type) [sorted rows, N / 2] = silu(gate) * up * row_w.  Tiles of 16 rows (what moe_sort was given).
CCB_API int ccb_moe_grouped(const void* A, int lda, const int* src_row, const void* W, int ldw,
                            long long w_expert_stride, void* C, int ldc, const float* row_w, const int* tile_e,
                            const int* tile_r0, const int* tile_n, int max_tiles, int N, int K, int BM, int mode,
                            int dtype, cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0) return 0;
  if (K <= 0 || mode < 0 || mode > 2 || (mode == 2 && (N & 1))) return CCB_REFUSE_SIZE;
  if (dtype == CCB_F32) {
    if (BM != 16) return CCB_REFUSE_SIZE;
    dim3 grid(max_tiles, (N + 127) / 128);
    if (mode == 2)
      ccb_launch(moe_grouped_f32_kernel<2>, grid, dim3(128), 0, stream, (const float*)A, lda, src_row, (const float*)W,
                 ldw, w_expert_stride, (float*)C, ldc, row_w, tile_e, tile_r0, tile_n, N, K);
    else if (mode == 0)
      ccb_launch(moe_grouped_f32_kernel<0>, grid, dim3(128), 0, stream, (const float*)A, lda, src_row, (const float*)W,
                 ldw, w_expert_stride, (float*)C, ldc, row_w, tile_e, tile_r0, tile_n, N, K);
    else
      ccb_launch(moe_grouped_f32_kernel<1>, grid, dim3(128), 0, stream, (const float*)A, lda, src_row, (const float*)W,
                 ldw, w_expert_stride, (float*)C, ldc, row_w, tile_e, tile_r0, tile_n, N, K);
    return ccb_launch_status();
  }
  if (dtype != CCB_BF16) return CCB_REFUSE_DTYPE;
  if (K % 8 || lda % 8 || ldw % 8 || w_expert_stride % 8 || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(W) & 15))
    return CCB_REFUSE_SIZE;
  // (tiles of more rows run on tcgen05: moe_tcgen05.cu.  An mma.sync form of this kernel for tiles of 32 and 64
  // rows, 128 columns a block, was measured against it and taken out: about twice as slow, 313 against 143 us
  // for the whole part at 128 tokens, 32 experts of 1536 x 4096 of which 4 are chosen)
  if (BM != 16) return CCB_REFUSE_SIZE;
  dim3 grid16((N + 7) / 8, max_tiles);   // the tiles that hold rows come first in the list, and so do their blocks
  if (mode == 2)
    ccb_launch(moe_grouped_rows16_kernel<2>, grid16, dim3(128), 0, stream, (const __nv_bfloat16*)A, lda, src_row,
               (const __nv_bfloat16*)W, ldw, w_expert_stride, C, ldc, row_w, tile_e, tile_r0, tile_n, N, K);
  else if (mode == 0)
    ccb_launch(moe_grouped_rows16_kernel<0>, grid16, dim3(128), 0, stream, (const __nv_bfloat16*)A, lda, src_row,
               (const __nv_bfloat16*)W, ldw, w_expert_stride, C, ldc, row_w, tile_e, tile_r0, tile_n, N, K);
  else
    ccb_launch(moe_grouped_rows16_kernel<1>, grid16, dim3(128), 0, stream, (const __nv_bfloat16*)A, lda, src_row,
               (const __nv_bfloat16*)W, ldw, w_expert_stride, C, ldc, row_w, tile_e, tile_r0, tile_n, N, K);
  return ccb_launch_status();
}

CCB_API int ccb_moe_combine(void* out, const float* rows, const int* pair_pos, const void* shared, int tokens, int top,
                            int D, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (top <= 0 || D <= 0) return CCB_REFUSE_SIZE;
  if (dtype != CCB_F32 && dtype != CCB_BF16) return CCB_REFUSE_DTYPE;
  if (D % 4 == 0 && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(rows) |
                      reinterpret_cast<uintptr_t>(shared)) & 15) == 0) {
    const size_t total4 = (size_t)tokens * (D / 4);
    const int blocks4 = (int)((total4 + 255) / 256 < 65535 * 8 ? (total4 + 255) / 256 : 65535 * 8);
    if (dtype == CCB_F32)
      ccb_launch(moe_combine_vec_kernel<float>, dim3(blocks4), dim3(256), 0, stream, (float*)out, rows, pair_pos,
                 (const float*)shared, top, D, total4);
    else
      ccb_launch(moe_combine_vec_kernel<__nv_bfloat16>, dim3(blocks4), dim3(256), 0, stream, (__nv_bfloat16*)out, rows,
                 pair_pos, (const __nv_bfloat16*)shared, top, D, total4);
    return ccb_launch_status();
  }
  const size_t total = (size_t)tokens * D;
  const int blocks = (int)((total + 255) / 256 < 65535 * 8 ? (total + 255) / 256 : 65535 * 8);
  if (dtype == CCB_F32)
    ccb_launch(moe_combine_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)out, rows, pair_pos,
               (const float*)shared, top, D, total);
  else if (dtype == CCB_BF16)
    ccb_launch(moe_combine_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)out, rows,
               pair_pos, (const __nv_bfloat16*)shared, top, D, total);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// act [rows, E F + shared] from gu [rows, 2 (E F + shared)] (gate columns, then up columns): see the kernel.
CCB_API int ccb_moe_dense_glu_act(void* act, int lda, const void* gu, int ldg, const float* dense_w,
                                  const float* shared_gate, int sg_stride, int rows, int E, int F, int shared,
                                  int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (E < 0 || F <= 0 || shared < 0 || lda < E * F + shared || ldg < 2 * (E * F + shared)) return CCB_REFUSE_SIZE;
  if (E > 0 && dense_w == nullptr) return CCB_REFUSE_ARG;
  const int width = E * F + shared;
  if (dtype == CCB_BF16 && (E == 0 || F % 8 == 0) && shared % 8 == 0 && lda % 8 == 0 && ldg % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(act) | reinterpret_cast<uintptr_t>(gu)) & 15) == 0) {
    const dim3 vgrid((width / 8 + 255) / 256, rows < 65535 ? rows : 65535);
    ccb_launch(moe_dense_glu_act_vec_kernel, vgrid, dim3(256), 0, stream, (__nv_bfloat16*)act, lda,
               (const __nv_bfloat16*)gu, ldg, dense_w, shared_gate, sg_stride, rows, E, F, shared);
    return ccb_launch_status();
  }
  const size_t total = (size_t)rows * (E * F + shared);
  const int blocks = (int)((total + 255) / 256 < 65535 * 8 ? (total + 255) / 256 : 65535 * 8);
  if (dtype == CCB_F32)
    ccb_launch(moe_dense_glu_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)act, lda, (const float*)gu,
               ldg, dense_w, shared_gate, sg_stride, rows, E, F, shared);
  else if (dtype == CCB_BF16)
    ccb_launch(moe_dense_glu_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)act, lda,
               (const __nv_bfloat16*)gu, ldg, dense_w, shared_gate, sg_stride, rows, E, F, shared);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}
