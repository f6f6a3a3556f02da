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
//
// Scores, mixing, maxima, sums and weights are float whatever the storage type.
#include "common.cuh"
#include <math_constants.h>

using namespace ccb;

namespace {

constexpr int kTalkWarps = 8;
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
        for (int i = 0; i < hd; i += 8) {
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
      for (int c = lane; c < hd; c += 32) {
        float acc = os[(size_t)h * hd + c] * corr;
        for (int kk = 0; kk < kTalkKeys; ++kk) {
          const float pk = pw[h * kTalkKeys + kk];
          const int vr = krows[kk];
          if (pk == 0.f || vr < 0) continue;   // the same for every lane
          acc = fmaf(pk, to_f32(v_cache[((size_t)vr + vhead) * hd + c]), acc);
        }
        os[(size_t)h * hd + c] = acc;
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

// out[t, h, :] = gate * sum_s acc_s exp(m_s - M) / (sum_s l_s exp(m_s - M) [+ exp(sink - M)]); a warp per (t, h).
template <typename T>
__global__ void attention_talking_merge_kernel(T* __restrict__ out, const float* __restrict__ part_acc,
                                               const float* __restrict__ part_ml, int rows, int nq, int hd,
                                               int num_splits, AttnExtra ex) {
  ccb::pdl_begin();
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= rows * nq) return;
  const int lane = threadIdx.x & 31;
  const int t = unit / nq, h = unit - t * nq;
  float M = -CUDART_INF_F;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, part_ml[(((size_t)t * num_splits + s) * nq + h) * 2]);
  T* orow = out + ((size_t)t * nq + h) * hd;
  if (M == -CUDART_INF_F) {
    for (int c = lane; c < hd; c += 32) orow[c] = from_f32<T>(0.f);
    return;
  }
  float ll = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float* pm = part_ml + (((size_t)t * num_splits + s) * nq + h) * 2;
    if (pm[0] != -CUDART_INF_F) ll += pm[1] * expf(pm[0] - M);
  }
  const float f = attn_sink_fold(ex, h, M, ll);
  const float mul = f * attn_gate<T>(ex, t, h) / ll;
  for (int c = lane; c < hd; c += 32) {
    float acc = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float ms = part_ml[(((size_t)t * num_splits + s) * nq + h) * 2];
      if (ms != -CUDART_INF_F) acc = fmaf(part_acc[(((size_t)t * num_splits + s) * nq + h) * hd + c], expf(ms - M), acc);
    }
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
  const int warps = 4;
  ccb_launch(attention_talking_merge_kernel<T>, dim3((rows * nq + warps - 1) / warps), dim3(warps * 32), 0, stream,
             (T*)out, (const float*)part_acc, (const float*)part_ml, rows, nq, hd, num_splits, ex);
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
  if (!ccb_attention_talking_fits(nq, nkv, hd) || page_size <= 0 || window < 0 || num_splits < 1 || num_splits > 65535)
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
