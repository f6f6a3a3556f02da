// Attention whose heads talk to each other before the softmax, over a paged cache.
//
// For a query at position p and a key at position j (p - window < j <= p, or every j <= p without a window):
//     r_g   = q_g . k_kv(g),j                         raw score of head g (kv(g) = g / (nq / nkv))
//     s_h   = sum_g M[h, g] r_g                       M [nq, nq]: the mixing matrix, with the score scale and any
//                                                     per-head temperature already multiplied into its columns
//     p_h   = softmax over the visible j of s_h       (optionally one more term exp(sink_h) in the denominator)
//     o_h   = gate_h * sum_j p_h,j v_kv(h),j          (optionally gate_h = sigmoid(gate logit of the token and head))
// Because every head's weights need every head's raw scores at the same (p, j), one block owns ALL heads of a query.
//
//   attention_talking         a block per query token, its warps dealing the heads among themselves.  32 keys at a
//                             time: each warp takes the raw scores of its heads (a lane per key, 16-byte loads of
//                             the key row), the block meets, each warp mixes the scores of its heads, updates their
//                             running maximum and sum and adds the weighted values (a lane per coordinate) into the
//                             heads' rows in shared memory.  With `num_splits` > 1 the key range of a token is cut
//                             into pieces, one block each, which leave (maximum, sum, unnormalised rows) per head;
//   attention_talking_merge   adds the pieces in a fixed order, folds the sink in and applies the gate.
//   attention_talking_mma     portions of prompts in bfloat16 (head size 64 or 128, at most 16 heads): a block owns 16
//                             neighbouring queries of a request and all heads, a warp per head.  32 keys at a time:
//                             every warp takes its head's raw scores on mma.sync (m16n8k16, the keys of all kv heads
//                             staged by cp.async, ldmatrix from swizzled rows) and leaves them in shared memory; after
//                             the block has met, every warp mixes its head's scores from all heads' raw ones (float),
//                             runs its softmax in the accumulator layout and multiplies the weights (rounded to
//                             bfloat16 as the operand, like the package's other tensor-core attention) with the staged
//                             values.  The next keys arrive while scores are mixed, the next values while raw scores
//                             are taken.  With 17 to 32 heads two blocks form a thread-block cluster: each owns half of
//                             the heads (and stages only their kv heads) and reads the other half's raw scores from
//                             its partner's shared memory (distributed shared memory) between two cluster barriers.
//
// Scores, mixing, maxima, sums and weights are float whatever the storage type.
#include "common.cuh"
#include "mma_common.cuh"
#include <cooperative_groups.h>
#include <math_constants.h>

using namespace ccb;

namespace {

constexpr int kTalkWarps = 16;   // (with 8 a warp had twice the heads, one after the other: 51 against 39 us a token,
                                 // merge included, at 32 heads of 128 over a window of 1,024)
constexpr int kTalkKeys = 32;

template <typename T> struct Row8;   // eight neighbouring elements of a row as floats
template <> struct Row8<float> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <> struct Row8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
};

template <typename T> struct Row4;   // four neighbouring elements as floats
template <> struct Row4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
template <> struct Row4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 a = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
  }
};

// q, out [T, nq, hd]; k_cache, v_cache [pages, nkv, page_size, hd]; mix float [nq, nq].
// part_acc [T, splits, nq, hd], part_ml [T, splits, nq, 2] (only with num_splits > 1).
template <typename T>
__global__ void __launch_bounds__(kTalkWarps * 32)
attention_talking_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                         T* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml,
                         const float* __restrict__ mix, const int* __restrict__ positions,
                         const int* __restrict__ entry_of_token, const int* __restrict__ block_table, int bt_stride,
                         int nq, int nkv, int hd, int page_size, int num_pages, int window, int num_splits,
                         AttnExtra ex, int* status) {
  ccb::pdl_begin();
  extern __shared__ __align__(16) float smem[];
  float* qs = smem;                                  // [nq, hd]
  float* os = qs + (size_t)nq * hd;                  // [nq, hd]
  float* ms = os + (size_t)nq * hd;                  // [nq, nq]
  float* raw = ms + (size_t)nq * nq;                 // [nq, 32]
  float* pw = raw + (size_t)nq * kTalkKeys;          // [nq, 32]
  float* run_m = pw + (size_t)nq * kTalkKeys;        // [nq]
  float* run_l = run_m + nq;                         // [nq]
  int* krows = reinterpret_cast<int*>(run_l + nq);   // [32]: the cache row of each key of the tile (-1: not seen)
  const int t = blockIdx.x, split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = entry_of_token[t];
  T* orow = out + (size_t)t * nq * hd;
  if (e < 0) {   // a row that pads a replayed step belongs to no request
    if (num_splits == 1)
      for (int i = threadIdx.x; i < nq * hd; i += blockDim.x) orow[i] = from_f32<T>(0.f);
    else
      for (int h = threadIdx.x; h < nq; h += blockDim.x) {
        part_ml[(((size_t)t * num_splits + split) * nq + h) * 2] = -CUDART_INF_F;
        part_ml[(((size_t)t * num_splits + split) * nq + h) * 2 + 1] = 0.f;
      }
    return;
  }
  const int p = positions[t];
  const int lo = first_visible_key(p, window, 0);
  // this block's share of the keys lo .. p: whole tiles of 32 keys counted from position 0
  const int tile_lo = lo / kTalkKeys, tile_hi = p / kTalkKeys;
  const int n_tiles = tile_hi - tile_lo + 1;
  const int per = (n_tiles + num_splits - 1) / num_splits;
  const int my_first = tile_lo + split * per;
  const int my_last = min(tile_hi, my_first + per - 1);
  const int* bt = block_table + (size_t)e * bt_stride;
  const int group = nq / nkv;

  const T* qrow = q + (size_t)t * nq * hd;
  for (int i = threadIdx.x; i < nq * hd; i += blockDim.x) {
    qs[i] = to_f32(qrow[i]);
    os[i] = 0.f;
  }
  for (int i = threadIdx.x; i < nq * nq; i += blockDim.x) ms[i] = mix[i];
  for (int h = threadIdx.x; h < nq; h += blockDim.x) {
    run_m[h] = -CUDART_INF_F;
    run_l[h] = 0.f;
  }
  __syncthreads();

  for (int tile = my_first; tile <= my_last; ++tile) {
    const int j = tile * kTalkKeys + lane;
    const bool seen = j >= lo && j <= p;
    // the row of this lane's key in the cache, without the kv head: (page * nkv) * page_size + place in the page
    int krow = -1;
    if (seen) {
      const int lp = j / page_size;
      const int page = lp < bt_stride ? bt[lp] : -1;
      if (page < 0 || page >= num_pages) set_status(status, CCB_ST_BAD_PAGE);
      else krow = page * nkv * page_size + (j - lp * page_size);
    }
    if (warp == 0) krows[lane] = krow;
    for (int g = warp; g < nq; g += kTalkWarps) {
      float s = 0.f;
      if (krow >= 0) {
        const T* kp = k_cache + ((size_t)krow + (size_t)(g / group) * page_size) * hd;
        const float* qg = qs + (size_t)g * hd;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll 8
        for (int i = 0; i < hd; i += 8) {   // (the loads of several rounds are in flight together)
          float kv[8];
          Row8<T>::load(kp + i, kv);
#pragma unroll
          for (int u = 0; u < 8; u += 2) {
            s0 = fmaf(qg[i + u], kv[u], s0);
            s1 = fmaf(qg[i + u + 1], kv[u + 1], s1);
          }
        }
        s = s0 + s1;
      }
      raw[g * kTalkKeys + lane] = s;
    }
    __syncthreads();   // every head's raw scores of the tile are there
    for (int h = warp; h < nq; h += kTalkWarps) {
      const float* mh = ms + (size_t)h * nq;
      float s = 0.f;
      for (int g = 0; g < nq; ++g) s = fmaf(mh[g], raw[g * kTalkKeys + lane], s);
      if (krow < 0) s = -CUDART_INF_F;
      const float m_old = run_m[h];
      const float m_new = fmaxf(m_old, warp_max(s));
      float pj = 0.f, corr = 1.f;
      if (m_new != -CUDART_INF_F) {
        pj = expf(s - m_new);          // 0 for a key that is not seen
        corr = expf(m_old - m_new);    // 0 the first time
      }
      const float l_new = run_l[h] * corr + warp_sum(pj);
      pw[h * kTalkKeys + lane] = pj;
      __syncwarp();
      if (lane == 0) {
        run_m[h] = m_new;
        run_l[h] = l_new;
      }
      const size_t vhead = (size_t)(h / group) * page_size;
      // four neighbouring coordinates a lane (a head of 128 is one pass of the warp over a value row).  A key that
      // is not seen has weight 0 and reads the first row of its kv head's first page instead: no branch stands
      // between the loads, so eight rows are in flight at a time
      for (int c = 4 * lane; c < hd; c += 128) {
        float4 acc = *reinterpret_cast<float4*>(os + (size_t)h * hd + c);
        acc.x *= corr; acc.y *= corr; acc.z *= corr; acc.w *= corr;
#pragma unroll 8
        for (int kk = 0; kk < kTalkKeys; ++kk) {
          const float pk = pw[h * kTalkKeys + kk];
          const int vr = krows[kk];
          const float4 vv = Row4<T>::load(v_cache + ((size_t)(vr < 0 ? 0 : vr) + vhead) * hd + c);
          acc.x = fmaf(pk, vv.x, acc.x);
          acc.y = fmaf(pk, vv.y, acc.y);
          acc.z = fmaf(pk, vv.z, acc.z);
          acc.w = fmaf(pk, vv.w, acc.w);
        }
        *reinterpret_cast<float4*>(os + (size_t)h * hd + c) = acc;
      }
      __syncwarp();
    }
    __syncthreads();   // the raw scores may be overwritten
  }

  if (num_splits > 1) {
    float* pa = part_acc + ((size_t)t * num_splits + split) * nq * hd;
    float* pm = part_ml + ((size_t)t * num_splits + split) * nq * 2;
    for (int i = threadIdx.x; i < nq * hd; i += blockDim.x) pa[i] = os[i];
    for (int h = threadIdx.x; h < nq; h += blockDim.x) {
      pm[2 * h] = run_m[h];
      pm[2 * h + 1] = run_l[h];
    }
    return;
  }
  for (int h = warp; h < nq; h += kTalkWarps) {
    float ll = run_l[h];
    const float f = attn_sink_fold(ex, h, run_m[h], ll);
    const float mul = ll > 0.f ? f * attn_gate<T>(ex, t, h) / ll : 0.f;
    for (int c = lane; c < hd; c += 32) orow[(size_t)h * hd + c] = from_f32<T>(os[(size_t)h * hd + c] * mul);
  }
}

// out[t, h, :] = gate * sum_s acc_s exp(m_s - M) / (sum_s l_s exp(m_s - M) [+ exp(sink - M)]); a block per (t, h):
// its first warp turns the pieces' maxima and sums into one weight per piece (at most 64 pieces), then every thread
// adds its coordinates over the pieces in their order.
constexpr int kMergeThreads = 128;
constexpr int kMaxSplits = 64;

template <typename T>
__global__ void __launch_bounds__(kMergeThreads)
attention_talking_merge_kernel(T* __restrict__ out, const float* __restrict__ part_acc,
                               const float* __restrict__ part_ml, int rows, int nq, int hd, int num_splits,
                               AttnExtra ex) {
  ccb::pdl_begin();
  __shared__ float wsplit[kMaxSplits];
  __shared__ float mul_s;
  const int t = blockIdx.x / nq, h = blockIdx.x - t * nq;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {
    float m[2], l[2];
    float M = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int sp = lane + 32 * i;
      m[i] = -CUDART_INF_F;
      l[i] = 0.f;
      if (sp < num_splits) {
        const float2 v = *reinterpret_cast<const float2*>(part_ml + (((size_t)t * num_splits + sp) * nq + h) * 2);
        m[i] = v.x;
        l[i] = v.y;
      }
      M = fmaxf(M, m[i]);
    }
    M = warp_max(M);
    float ll = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float wgt = (m[i] == -CUDART_INF_F) ? 0.f : expf(m[i] - M);
      if (lane + 32 * i < kMaxSplits) wsplit[lane + 32 * i] = wgt;
      ll += l[i] * wgt;
    }
    ll = warp_sum(ll);
    if (lane == 0) {
      float mul = 0.f;
      if (M != -CUDART_INF_F) {
        const float f = attn_sink_fold(ex, h, M, ll);
        mul = f * attn_gate<T>(ex, t, h) / ll;
      }
      mul_s = mul;
    }
  }
  __syncthreads();
  const float mul = mul_s;
  T* orow = out + ((size_t)t * nq + h) * hd;
  for (int c = threadIdx.x; c < hd; c += kMergeThreads) {
    float acc = 0.f;
#pragma unroll 8
    for (int sp = 0; sp < num_splits; ++sp)
      acc = fmaf(part_acc[(((size_t)t * num_splits + sp) * nq + h) * hd + c], wsplit[sp], acc);
    orow[c] = from_f32<T>(acc * mul);
  }
}

size_t talking_smem(int nq, int hd) {
  return ((size_t)2 * nq * hd + (size_t)nq * nq + (size_t)2 * nq * kTalkKeys + 2 * (size_t)nq + kTalkKeys) * sizeof(float);
}

template <typename T>
int launch_talking(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_acc,
                   float* part_ml, const float* mix, const int* positions, const int* entry_of_token,
                   const int* block_table, int bt_stride, int rows, int nq, int nkv, int hd, int page_size,
                   int num_pages, int window, int num_splits, AttnExtra ex, int* status, cudaStream_t stream) {
  const size_t smem = talking_smem(nq, hd);
  cudaFuncSetAttribute(attention_talking_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  ccb_launch(attention_talking_kernel<T>, dim3(rows, num_splits), dim3(kTalkWarps * 32), smem, stream, (const T*)q,
             (const T*)k_cache, (const T*)v_cache, (T*)out, part_acc, part_ml, mix, positions, entry_of_token,
             block_table, bt_stride, nq, nkv, hd, page_size, num_pages, window, num_splits, ex, status);
  int rc = ccb_launch_status();
  if (rc != 0 || num_splits == 1) return rc;
  ccb_launch(attention_talking_merge_kernel<T>, dim3(rows * nq), dim3(kMergeThreads), 0, stream, (T*)out,
             (const float*)part_acc, (const float*)part_ml, rows, nq, hd, num_splits, ex);
  return ccb_launch_status();
}


// ---------------------------------------------------------------------------------------------
// Portions of prompts on tensor cores (bfloat16).  See the head of the file.
constexpr int kMmaQ = 16;       // queries of a block
constexpr int kMmaKeys = 32;    // keys staged at a time
constexpr int kRawLd = 36;      // floats of a row of raw scores.  A thread's eight values of a row (its two columns of
                                // each of the four 8-key blocks) lie side by side, at 8 tig + 2 block + e, and are
                                // moved 16 bytes at a time; with 32 + 4 floats a row the eight threads of such an
                                // access (two rows, four tig) fall into different banks

template <int HD, int CL>
__global__ void __launch_bounds__(512)
attention_talking_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                             const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out,
                             const float* __restrict__ mix, const int* __restrict__ cu_q,
                             const int* __restrict__ pos0, const int* __restrict__ block_table, int bt_stride,
                             int entry0, int nq, int nkv, int page_size, int num_pages, int window, AttnExtra ex,
                             int* status) {
  ccb::pdl_begin();
  constexpr int KS = HD / 16;   // k-steps over a head
  constexpr int CH = HD / 8;    // 16-byte chunks of a row
  extern __shared__ __align__(128) unsigned char smem_raw[];
  namespace cg = cooperative_groups;
  // the block's heads: all of them, or with a cluster of CL blocks the rank's share (and their kv heads)
  const int hpc = nq / CL, kv_local = nkv / CL;
  int rank = 0;
  if constexpr (CL > 1) rank = (int)cg::this_cluster().block_rank();
  __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);               // [kv_local][32][HD], swizzled rows
  __nv_bfloat16* v_s = k_s + (size_t)kv_local * kMmaKeys * HD;                   // the same for the values
  float* raw = reinterpret_cast<float*>(v_s + (size_t)kv_local * kMmaKeys * HD);  // [hpc][16][kRawLd]
  float* ms = raw + (size_t)hpc * kMmaQ * kRawLd;                                 // [hpc][nq]: the rows of its heads
  // In a cluster of two: a copy of the partner's raw scores of the tile.  They are fetched once a tile, 16 bytes a
  // thread and access, rather than read in place by every warp (distributed shared memory is far slower than a
  // block's own: with the partner's scores read in place the kernel took 3.4 times as long at 32 heads of 128).
  float* partner_copy = ms + (size_t)hpc * nq;                                    // [hpc][16][kRawLd], CL == 2 only
  const float* raw_of[CL];   // where this block reads the raw scores of each block's heads
  const float* partner_raw = nullptr;
  raw_of[0] = raw;
  if constexpr (CL > 1) {
    static_assert(CL == 2, "a cluster of two");
    partner_raw = cg::this_cluster().map_shared_rank(raw, rank ^ 1);
    raw_of[rank] = raw;
    raw_of[rank ^ 1] = partner_copy;
  }

  const int b = entry0 + blockIdx.y;
  const int row_begin = cu_q[b], n_new = cu_q[b + 1] - row_begin;
  const int n_qtiles = (n_new + kMmaQ - 1) / kMmaQ;
  const int qt = n_qtiles - 1 - (int)blockIdx.x / CL;   // long tiles first (the blocks of a cluster share a tile)
  if (qt < 0) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = rank * hpc + warp;                              // a warp per head
  const int gid = lane >> 2, tig = lane & 3;
  const int kvh = h / (nq / nkv) - rank * kv_local;             // among the kv heads staged here
  const int q_first = qt * kMmaQ;
  const int rows_here = min(kMmaQ, n_new - q_first);
  const int p_first = pos0[b] + q_first, p_last = p_first + rows_here - 1;
  const int* bt = block_table + (size_t)b * bt_stride;
  const int j_lo = first_visible_key(p_first, window, 0);
  const int first_tile = j_lo / kMmaKeys, n_tiles = p_last / kMmaKeys - first_tile + 1;
  const int n_threads = hpc * 32;

  // (the mixing matrix times log2(e): the softmax runs on base-2 exponentials, one instruction each)
  for (int i = tid; i < hpc * nq; i += n_threads) ms[i] = mix[(size_t)rank * hpc * nq + i] * 1.4426950408889634f;

  // this head's query rows as A fragments, straight from global memory (rows beyond the portion are zero)
  uint32_t qa[KS][4];
  {
    const bool ok0 = gid < rows_here, ok1 = gid + 8 < rows_here;
    const __nv_bfloat16* q0 = q + ((size_t)(row_begin + q_first + (ok0 ? gid : 0)) * nq + h) * HD + 2 * tig;
    const __nv_bfloat16* q1 = q + ((size_t)(row_begin + q_first + (ok1 ? gid + 8 : 0)) * nq + h) * HD + 2 * tig;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qa[ks][0] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + 16 * ks) : 0u;
      qa[ks][1] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + 16 * ks) : 0u;
      qa[ks][2] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + 16 * ks + 8) : 0u;
      qa[ks][3] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + 16 * ks + 8) : 0u;
    }
  }

  // a tile of keys (or values) of every kv head: row r = kv head * 32 + key, its 16-byte chunks swizzled
  const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
  auto issue = [&](const __nv_bfloat16* cache, __nv_bfloat16* dst, int tile) {
    for (int i = tid; i < kMmaKeys * CH; i += n_threads) {   // (key of the tile, chunk): the page is looked up once
      const int kr = i / CH, c = i - kr * CH;
      const int j = tile * kMmaKeys + kr;
      bool valid = j >= j_lo && j <= p_last;
      size_t src = 0;
      if (valid) {
        const int lp = page_shift >= 0 ? (j >> page_shift) : (j / page_size);
        const int page = lp < bt_stride ? bt[lp] : -1;
        if (page < 0 || page >= num_pages) {
          set_status(status, CCB_ST_BAD_PAGE);
          valid = false;
        } else {
          src = (((size_t)page * nkv + rank * kv_local) * page_size + (j - lp * page_size)) * HD + c * 8;
        }
      }
      const uint32_t d0 = smem_u32(dst + swz<HD>(kr, c));   // (32 rows a kv head: the swizzle is the same for each)
      const size_t head_stride = (size_t)page_size * HD;
      for (int kh = 0; kh < kv_local; ++kh)
        cp_async16(d0 + (uint32_t)(kh * kMmaKeys * HD * 2), cache + src + kh * head_stride, valid);
    }
  };

  const int pr0 = p_first + gid, pr1 = pr0 + 8;
  const int lo0 = first_visible_key(pr0, window, 0), lo1 = first_visible_key(pr1, window, 0);
  const bool live0 = gid < rows_here, live1 = gid + 8 < rows_here;
  const int lo_last = first_visible_key(p_last, window, 0);   // (the first key that the block's last row sees)

  float o[2 * KS][4];
#pragma unroll
  for (int i = 0; i < 2 * KS; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

  issue(k_cache, k_s, first_tile);
  cp_async_commit();
  const float* mh = ms + (size_t)warp * nq;
  float* my_raw = raw + (size_t)warp * kMmaQ * kRawLd;
  const __nv_bfloat16* k_h = k_s + (size_t)kvh * kMmaKeys * HD;
  const __nv_bfloat16* v_h = v_s + (size_t)kvh * kMmaKeys * HD;

  for (int it = 0; it < n_tiles; ++it) {
    const int jt = (first_tile + it) * kMmaKeys;
    cp_async_wait<0>();
    // the keys of this tile are there; everybody is done with the values of the tile before (and, in a cluster,
    // the partner is done with this block's raw scores of the tile before)
    if constexpr (CL > 1) cg::this_cluster().sync(); else __syncthreads();
    issue(v_cache, v_s, first_tile + it);
    cp_async_commit();
    // raw scores of this head: S [16 x 32] = Q K^T
    float sc[4][4];
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.f;
    {
      const int krow = (lane & 7) + 8 * (lane >> 4);
      const int kchunk = (lane >> 3) & 1;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b00, b01, b10, b11;
          ldmatrix_x4(b00, b01, b10, b11, smem_u32(k_h + swz<HD>(np * 16 + krow, 2 * ks + kchunk)));
          mma_bf16_16816(sc[2 * np], qa[ks], b00, b01);
          mma_bf16_16816(sc[2 * np + 1], qa[ks], b10, b11);
        }
      }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float* r0p = my_raw + gid * kRawLd + 8 * tig + 4 * half;
      float* r1p = my_raw + (gid + 8) * kRawLd + 8 * tig + 4 * half;
      *reinterpret_cast<float4*>(r0p) = make_float4(sc[2 * half][0], sc[2 * half][1], sc[2 * half + 1][0], sc[2 * half + 1][1]);
      *reinterpret_cast<float4*>(r1p) = make_float4(sc[2 * half][2], sc[2 * half][3], sc[2 * half + 1][2], sc[2 * half + 1][3]);
    }
    // every head's raw scores are there (in a cluster: the partner's too); the keys' buffer is free
    if constexpr (CL > 1) cg::this_cluster().sync(); else __syncthreads();
    if (it + 1 < n_tiles) issue(k_cache, k_s, first_tile + it + 1);
    cp_async_commit();
    if constexpr (CL > 1) {
      const float4* src = reinterpret_cast<const float4*>(partner_raw);
      float4* dst = reinterpret_cast<float4*>(partner_copy);
      for (int i = tid; i < hpc * kMmaQ * kRawLd / 4; i += n_threads) dst[i] = src[i];
      __syncthreads();
    }
    // this head's scores: the mix of all heads' raw ones (float), in the accumulator's layout
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.f;
#pragma unroll
    for (int r = 0; r < CL; ++r) {
      const float* rg = raw_of[r] + gid * kRawLd + 8 * tig;
      const float* mr = mh + r * hpc;
#pragma unroll 4
      for (int g = 0; g < hpc; ++g, rg += kMmaQ * kRawLd) {
        const float wgt = mr[g];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const float4 a = *reinterpret_cast<const float4*>(rg + 4 * half);
          const float4 c = *reinterpret_cast<const float4*>(rg + 8 * kRawLd + 4 * half);
          sc[2 * half][0] = fmaf(wgt, a.x, sc[2 * half][0]);
          sc[2 * half][1] = fmaf(wgt, a.y, sc[2 * half][1]);
          sc[2 * half + 1][0] = fmaf(wgt, a.z, sc[2 * half + 1][0]);
          sc[2 * half + 1][1] = fmaf(wgt, a.w, sc[2 * half + 1][1]);
          sc[2 * half][2] = fmaf(wgt, c.x, sc[2 * half][2]);
          sc[2 * half][3] = fmaf(wgt, c.y, sc[2 * half][3]);
          sc[2 * half + 1][2] = fmaf(wgt, c.z, sc[2 * half + 1][2]);
          sc[2 * half + 1][3] = fmaf(wgt, c.w, sc[2 * half + 1][3]);
        }
      }
    }
    float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
    // a tile that every row of the block sees whole needs no mask (the same for all threads)
    const bool inside = rows_here == kMmaQ && jt + kMmaKeys - 1 <= p_first && jt >= lo_last;
    if (!inside) {
#pragma unroll
      for (int nb = 0; nb < 4; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = jt + nb * 8 + 2 * tig + e;
          sc[nb][e] = (live0 && j <= pr0 && j >= lo0) ? sc[nb][e] : -CUDART_INF_F;
          sc[nb][2 + e] = (live1 && j <= pr1 && j >= lo1) ? sc[nb][2 + e] : -CUDART_INF_F;
        }
    }
#pragma unroll
    for (int nb = 0; nb < 4; ++nb)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        mx0 = fmaxf(mx0, sc[nb][e]);
        mx1 = fmaxf(mx1, sc[nb][2 + e]);
      }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float c0 = mn0 == -CUDART_INF_F ? 1.f : exp2f(m0 - mn0);
    const float c1 = mn1 == -CUDART_INF_F ? 1.f : exp2f(m1 - mn1);
    const float sub0 = mn0 == -CUDART_INF_F ? 0.f : mn0, sub1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
    m0 = mn0;
    m1 = mn1;
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int nb = 0; nb < 4; ++nb)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        sc[nb][e] = exp2f(sc[nb][e] - sub0);
        sc[nb][2 + e] = exp2f(sc[nb][2 + e] - sub1);
        ps0 += sc[nb][e];
        ps1 += sc[nb][2 + e];
      }
    l0 = l0 * c0 + ps0;
    l1 = l1 * c1 + ps1;
#pragma unroll
    for (int i = 0; i < 2 * KS; ++i) {
      o[i][0] *= c0; o[i][1] *= c0;
      o[i][2] *= c1; o[i][3] *= c1;
    }
    cp_async_wait<1>();   // the values (the keys of the next tile may still be on their way)
    __syncthreads();
    {
      const int vrow = (lane & 7) + 8 * ((lane >> 3) & 1);
      const int vchunk = lane >> 4;
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {   // 16 keys at a time
        uint32_t pa[4];
        pa[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
        pa[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
        pa[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
        pa[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
        for (int nn = 0; nn < KS; ++nn) {
          uint32_t b00, b01, b10, b11;
          ldmatrix_x4_trans(b00, b01, b10, b11, smem_u32(v_h + swz<HD>(kk * 16 + vrow, 2 * nn + vchunk)));
          mma_bf16_16816(o[2 * nn], pa, b00, b01);
          mma_bf16_16816(o[2 * nn + 1], pa, b10, b11);
        }
      }
    }
  }
  cp_async_wait<0>();
  if constexpr (CL > 1) cg::this_cluster().sync();   // (the partner may still be reading this block's raw scores)
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  float f0 = 1.f, f1 = 1.f;
  if (ex.sink != nullptr) {   // one more term in each denominator (the maxima are in the base-2 scale of the scores)
    const float sk = ex.sink[h] * 1.4426950408889634f;
    const float n0 = fmaxf(m0, sk), n1 = fmaxf(m1, sk);
    f0 = m0 == -CUDART_INF_F ? 0.f : exp2f(m0 - n0);
    f1 = m1 == -CUDART_INF_F ? 0.f : exp2f(m1 - n1);
    l0 = l0 * f0 + exp2f(sk - n0);
    l1 = l1 * f1 + exp2f(sk - n1);
  }
  float inv0 = l0 > 0.f ? f0 / l0 : 0.f, inv1 = l1 > 0.f ? f1 / l1 : 0.f;
  if (live0) inv0 *= attn_gate<__nv_bfloat16>(ex, row_begin + q_first + gid, h);
  if (live1) inv1 *= attn_gate<__nv_bfloat16>(ex, row_begin + q_first + gid + 8, h);
  __nv_bfloat16* o0 = out + ((size_t)(row_begin + q_first + gid) * nq + h) * HD;
  __nv_bfloat16* o1 = out + ((size_t)(row_begin + q_first + gid + 8) * nq + h) * HD;
#pragma unroll
  for (int i = 0; i < 2 * KS; ++i) {
    const int d = i * 8 + 2 * tig;
    if (live0) *reinterpret_cast<uint32_t*>(o0 + d) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
    if (live1) *reinterpret_cast<uint32_t*>(o1 + d) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
  }
}

int talking_mma_cluster(int nq) { return nq <= 16 ? 1 : 2; }

size_t talking_mma_smem(int nq, int nkv, int hd) {
  const int cl = talking_mma_cluster(nq);
  return (size_t)2 * (nkv / cl) * kMmaKeys * hd * sizeof(__nv_bfloat16) +
         (size_t)cl * (nq / cl) * kMmaQ * kRawLd * sizeof(float) + (size_t)(nq / cl) * nq * sizeof(float);
}

template <int HD, int CL>
int launch_talking_mma(const void* q, const void* k_cache, const void* v_cache, void* out, const float* mix,
                       const int* cu_q, const int* pos0, const int* block_table, int bt_stride, int entry0,
                       int n_entries, int max_new, int nq, int nkv, int page_size, int num_pages, int window,
                       AttnExtra ex, int* status, cudaStream_t stream) {
  const size_t smem = talking_mma_smem(nq, nkv, HD);
  cudaError_t e = cudaFuncSetAttribute(attention_talking_mma_kernel<HD, CL>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(CL * ((max_new + kMmaQ - 1) / kMmaQ), n_entries);
  if (CL == 1) {
    ccb_launch(attention_talking_mma_kernel<HD, CL>, grid, dim3(nq * 32), smem, stream, (const __nv_bfloat16*)q,
               (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out, mix, cu_q, pos0,
               block_table, bt_stride, entry0, nq, nkv, page_size, num_pages, window, ex, status);
    return ccb_launch_status();
  }
  // a cluster of CL neighbouring blocks along x
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(nq / CL * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, attention_talking_mma_kernel<HD, CL>, (const __nv_bfloat16*)q,
                     (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out, mix, cu_q, pos0,
                     block_table, bt_stride, entry0, nq, nkv, page_size, num_pages, window, ex, status);
  return ccb_launch_status();
}

}  // namespace

// Whether the kernel takes these sizes (its shared memory holds every head's query and result rows).
CCB_API int ccb_attention_talking_fits(int nq, int nkv, int hd) {
  return nq > 0 && nkv > 0 && nq % nkv == 0 && hd > 0 && hd % 8 == 0 && talking_smem(nq, hd) <= 200 * 1024;
}

CCB_API int ccb_attention_talking(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_acc,
                                  float* part_ml, const float* mix, const int* positions, const int* entry_of_token,
                                  const int* block_table, int bt_stride, int rows, int nq, int nkv, int hd,
                                  int page_size, int num_pages, int window, int num_splits, const float* sink,
                                  const void* gate, int gate_stride, int dtype, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!ccb_attention_talking_fits(nq, nkv, hd) || page_size <= 0 || window < 0 || num_splits < 1 || num_splits > kMaxSplits)
    return CCB_REFUSE_SIZE;
  if (mix == nullptr || (num_splits > 1 && (part_acc == nullptr || part_ml == nullptr))) return CCB_REFUSE_ARG;
  AttnExtra ex{0, sink, gate, gate_stride};
  if (dtype == CCB_F32)
    return launch_talking<float>(q, k_cache, v_cache, out, part_acc, part_ml, mix, positions, entry_of_token,
                                 block_table, bt_stride, rows, nq, nkv, hd, page_size, num_pages, window, num_splits,
                                 ex, status, stream);
  if (dtype == CCB_BF16)
    return launch_talking<__nv_bfloat16>(q, k_cache, v_cache, out, part_acc, part_ml, mix, positions, entry_of_token,
                                         block_table, bt_stride, rows, nq, nkv, hd, page_size, num_pages, window,
                                         num_splits, ex, status, stream);
  return CCB_REFUSE_DTYPE;
}

// The tensor-core form for portions of prompts: bfloat16, head size 64 or 128, at most 16 heads a block (a warp
// each) and at most two blocks a cluster (then heads and kv heads split in two), and shared memory for a tile of
// keys and of values of the block's kv heads.
CCB_API int ccb_attention_talking_mma_fits(int nq, int nkv, int hd) {
  if (!(nq > 0 && nq <= 32 && nkv > 0 && nq % nkv == 0 && (hd == 64 || hd == 128))) return 0;
  const int cl = talking_mma_cluster(nq);
  if (nq % cl || nkv % cl) return 0;
  return talking_mma_smem(nq, nkv, hd) <= 220 * 1024;
}

// Requests entry0 .. entry0 + n_entries - 1 of the step (none with more than max_new tokens); bfloat16.
CCB_API int ccb_attention_talking_mma(const void* q, const void* k_cache, const void* v_cache, void* out,
                                      const float* mix, const int* cu_q, const int* pos0, const int* block_table,
                                      int bt_stride, int entry0, int n_entries, int max_new, int nq, int nkv, int hd,
                                      int page_size, int num_pages, int window, const float* sink, const void* gate,
                                      int gate_stride, int* status, cudaStream_t stream) {
  if (n_entries <= 0 || max_new <= 0) return 0;
  if (!ccb_attention_talking_mma_fits(nq, nkv, hd) || page_size <= 0 || window < 0 || n_entries > 65535)
    return CCB_REFUSE_SIZE;
  if (mix == nullptr || (gate != nullptr && gate_stride < nq)) return CCB_REFUSE_ARG;
  AttnExtra ex{0, sink, gate, gate_stride};
#define CCB_TALK_MMA(HD_, CL_)                                                                                       \
  launch_talking_mma<HD_, CL_>(q, k_cache, v_cache, out, mix, cu_q, pos0, block_table, bt_stride, entry0, n_entries, \
                               max_new, nq, nkv, page_size, num_pages, window, ex, status, stream)
  const int cl = talking_mma_cluster(nq);
  if (hd == 128) return cl == 1 ? CCB_TALK_MMA(128, 1) : CCB_TALK_MMA(128, 2);
  return cl == 1 ? CCB_TALK_MMA(64, 1) : CCB_TALK_MMA(64, 2);
#undef CCB_TALK_MMA
}
