// Latent attention: softmax attention whose keys and values are all made from ONE low-rank vector per token.
//
// Per token the layer keeps c (rank R, an RMS-normed projection of the input) and kr (r coordinates, rotated by
// the position, shared by all heads).  Head h has  key_j = [Wuk_h c_j | kr_j]  and  value_j = Wuv_h c_j, so
//   score_ij = (qu_i . Wuk_h c_j + qr_i . kr_j) * scale = ((Wuk_h^T qu_i) . c_j + qr_i . kr_j) * scale
//   out_i    = Wuv_h (sum_j p_ij c_j)
// and attention runs over the cached rows [c | kr] themselves, every head reading the same row: the query is
// carried into the latent space first (a product per head, done by the caller), the weighted sum of c comes
// back out through Wuv_h afterwards.  A query at position p sees the keys p - window + 1 .. p.  The softmax has
// one more term per head, exp(sink_h), with no key and no value (it starts the running maximum and sum).
// Each head's result is multiplied by sigmoid(gate logit of the head) before it is written.
//
// Two kernels:
//   latent_prepare    a block per token: c = x / rms(x) * w and kr = rot(x') into the cache row of the token;
//                     the rotated part of every head's query into the query rows [T, H, R + r] (float)
//   latent_attention  a block per (run of `tq` query tokens of a request, group of heads): 32 cached rows at
//                     a time are staged in shared memory as floats; a warp owns one (query, head): a lane
//                     takes a key for the scores, then a slice of the coordinates for the weighted sum
//
// Scores, weights, sums and the rotation are float whatever the storage type.
#include "common.cuh"
#include "mma_common.cuh"
#include <math_constants.h>

using namespace ccb;

namespace {

constexpr int kPrepThreads = 128;

// proj [T, ld]: columns q at oq (H heads of [d | r]) and the latent row at oc ([R | r]).
// cache [slots, R + r]; qa [T, H, R + r] float (only the last r of each head are written here).
template <typename T>
__global__ void __launch_bounds__(kPrepThreads)
latent_prepare_kernel(const T* __restrict__ proj, int ld, int oq, int oc, const float* __restrict__ w,
                      const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ positions,
                      const int* __restrict__ slot_map, T* __restrict__ cache, int num_slots, float* __restrict__ qa,
                      int H, int d, int r, int R, float eps, int* status) {
  ccb::pdl_begin();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int pos = positions[t];
  const T* row = proj + (size_t)t * ld;
  const int half = rot_dims >> 1;
  const int slot = slot_map ? slot_map[t] : -1;
  const bool keep = slot >= 0;
  // the token's blocks share the work: block 0 of the row makes the cache row, the others the queries' rotated
  // parts (all of it in one block when the grid has one block a token)
  const int parts = gridDim.y;
  if (blockIdx.y == 0 && keep && slot >= num_slots) set_status(status, CCB_ST_BAD_SLOT);
  if (blockIdx.y == 0 && keep && slot < num_slots) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += kPrepThreads) {
      const float v = to_f32(row[oc + i]);
      ss += v * v;
    }
    ss = block_sum<kPrepThreads>(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)R + eps);
    T* dst = cache + (size_t)slot * (R + r);
    for (int i = threadIdx.x; i < R; i += kPrepThreads) dst[i] = from_f32<T>(to_f32(row[oc + i]) * inv * w[i]);
    const T* kr = row + oc + R;
    for (int i = threadIdx.x; i < r; i += kPrepThreads) {
      float v;
      if (i < rot_dims) {
        const int j = i < half ? i : i - half;
        float sn, cs;
        sincosf((float)pos * inv_freq[j], &sn, &cs);
        const float a = to_f32(kr[j]), b = to_f32(kr[j + half]);
        v = i < half ? a * cs - b * sn : b * cs + a * sn;
      } else {
        v = to_f32(kr[i]);
      }
      dst[R + i] = from_f32<T>(v);
    }
  }
  const int q_total = H * r;
  const int q_per = parts > 1 ? (q_total + parts - 2) / (parts - 1) : q_total;
  const int q_lo = (parts > 1 && blockIdx.y > 0) ? ((int)blockIdx.y - 1) * q_per : 0;
  const int q_hi = parts > 1 ? (blockIdx.y == 0 ? 0 : min(q_total, q_lo + q_per)) : q_total;
  for (int i = q_lo + threadIdx.x; i < q_hi; i += kPrepThreads) {
    const int h = i / r, k = i - h * r;
    const T* qr = row + oq + (size_t)h * (d + r) + d;
    float v;
    if (k < rot_dims) {
      const int j = k < half ? k : k - half;
      float sn, cs;
      sincosf((float)pos * inv_freq[j], &sn, &cs);
      const float a = to_f32(qr[j]), b = to_f32(qr[j + half]);
      v = k < half ? a * cs - b * sn : b * cs + a * sn;
    } else {
      v = to_f32(qr[k]);
    }
    qa[((size_t)t * H + h) * (R + r) + R + k] = v;
  }
}

constexpr int kAttWarps = 8;
constexpr int kKeys = 32;   // cached rows staged at a time

// NV: coordinates of c per lane (R <= 32 NV).
// Shared memory: tile [kKeys][LD] floats (LD odd: a lane per row reads without bank conflicts), then the
// queries of the block's warps [kAttWarps][R + r].
template <typename T, int NV>
__global__ void __launch_bounds__(kAttWarps * 32)
latent_attention_kernel(const float* __restrict__ qa, const T* __restrict__ cache, const float* __restrict__ sink,
                        const T* __restrict__ gate, int ldg, T* __restrict__ out, const int* __restrict__ cu_q,
                        const int* __restrict__ pos0, const int* __restrict__ entry_of_token, const int* __restrict__ block_table, int bt_stride, int entry0,
                        int H, int R, int r, int page_size, int num_pages, int window, float scale, int tq,
                        int* status) {
  ccb::pdl_begin();
  extern __shared__ __align__(16) float smem[];
  const int W = R + r;
  const int LD = W | 1;
  float* tile = smem;
  float* qs = smem + (size_t)kKeys * LD;
  const int e = entry0 + blockIdx.z;
  const int r0 = cu_q[e], n = cu_q[e + 1] - r0;
  const int qbase = blockIdx.x * tq;
  if (qbase >= n || entry_of_token[r0 + qbase] < 0) return;   // (rows that pad a replayed step belong to no request)
  const int hg = kAttWarps / tq;   // heads per block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qi = warp / hg, head = blockIdx.y * hg + (warp - qi * hg);
  const bool live = qbase + qi < n && head < H;
  const int p_first = pos0[e] + qbase;
  const int p_last = p_first + min(tq, n - qbase) - 1;
  const int p = p_first + qi;                     // this warp's position
  const int t = r0 + qbase + qi;                  // and token row
  const int j_lo = max(0, p_first - window + 1);
  const int my_lo = max(0, p - window + 1);
  const int* bt = block_table + (size_t)e * bt_stride;

  float* q = qs + (size_t)warp * W;
  if (live) {
    const float* src = qa + ((size_t)t * H + head) * W;
    for (int i = lane; i < W; i += 32) q[i] = src[i];
  }
  float m = live ? sink[head] : 0.f, l = 1.f;   // the sink: one term exp(sink) with no key and no value
  float acc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) acc[i] = 0.f;

  for (int j0 = j_lo & ~(kKeys - 1); j0 <= p_last; j0 += kKeys) {
    __syncthreads();   // the tile of the round before has been read (and, the first time, q is written)
    for (int rr = warp; rr < kKeys; rr += kAttWarps) {
      const int j = j0 + rr;
      float* dst = tile + (size_t)rr * LD;
      const T* src = nullptr;
      if (j >= j_lo && j <= p_last) {
        const int lp = j / page_size;
        const int page = lp < bt_stride ? bt[lp] : -1;
        if (page < 0 || page >= num_pages) set_status(status, CCB_ST_BAD_PAGE);
        else src = cache + ((size_t)page * page_size + (j - lp * page_size)) * W;
      }
      if (src) for (int i = lane; i < W; i += 32) dst[i] = to_f32(src[i]);
      else for (int i = lane; i < W; i += 32) dst[i] = 0.f;
    }
    __syncthreads();
    if (!live) continue;
    const int j = j0 + lane;
    const float* kj = tile + (size_t)lane * LD;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    int i = 0;
    for (; i + 3 < W; i += 4) {
      s0 = fmaf(q[i], kj[i], s0);
      s1 = fmaf(q[i + 1], kj[i + 1], s1);
      s2 = fmaf(q[i + 2], kj[i + 2], s2);
      s3 = fmaf(q[i + 3], kj[i + 3], s3);
    }
    for (; i < W; ++i) s0 = fmaf(q[i], kj[i], s0);
    float s = ((s0 + s1) + (s2 + s3)) * scale;
    if (j < my_lo || j > p) s = -CUDART_INF_F;
    const float m_new = fmaxf(m, warp_max(s));   // finite: m starts at the sink
    const float corr = expf(m - m_new);
    const float pj = expf(s - m_new);            // 0 for a key that is not seen
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int v = 0; v < NV; ++v) acc[v] *= corr;
    for (int k = 0; k < kKeys; ++k) {
      const float pk = __shfl_sync(0xffffffffu, pj, k);
      if (pk == 0.f) continue;                   // the same for every lane
      const float* ck = tile + (size_t)k * LD;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int c = lane + 32 * v;
        if (c < R) acc[v] = fmaf(pk, ck[c], acc[v]);
      }
    }
  }
  if (!live) return;
  const float g = gate ? 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * ldg + head]))) : 1.0f;   // (no gate: the factor is one)
  const float f = g / l;
  T* dst = out + ((size_t)t * H + head) * R;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int c = lane + 32 * v;
    if (c < R) dst[c] = from_f32<T>(acc[v] * f);
  }
}

// ---------------------------------------------------------------------------------------------
// The same attention on tensor cores (bfloat16; R and r multiples of 16, R <= 512).
//
// All heads read the same cached rows, so the heads are the rows of the products: a block owns 16 rows, the
// (query, head) pairs of hpb heads x 16 / hpb neighbouring queries, and walks the keys 32 at a time:
//   S [16 x 32] = Q [16 x (R + r)] C^T        mma.sync m16n8k16; warp w takes the tile's keys 8 w .. 8 w + 7 over
//                                              the whole width, Q and the keys from shared memory by ldmatrix
//   softmax over the 32 keys                   float; maxima and sums meet in shared memory; P in bfloat16
//   O [16 x R] += P [16 x 32] C [32 x R]       warp w takes the columns 16 (w + 4 i) .. + 15, keys by ldmatrix.trans
// The cached rows arrive by cp.async, the next 32 while the current ones are used.  With few rows the key range
// of a row is cut into `num_splits` pieces, one block each; a second kernel merges the pieces (the sink counts
// in piece 0).  Rows of shared memory are 16 bytes longer than their data, so that the eight rows an ldmatrix
// reads fall into different banks.
constexpr int kMmaWarps = 4;   // of a block of single tokens

// MTL: tiles of 16 rows a block; WARPS: the warps of one tile of rows, each with 8 of the 8 * WARPS keys staged at
// a time (a block has MTL * WARPS warps: warp (rt, wk) owns the tile of rows rt and the keys / columns of wk).
// Single tokens: 16 rows, 4 warps, 32 keys (two blocks an SM).  Portions of prompts: 32 rows, 16 warps, 64 keys
// (one block an SM): twice the queries share every staged key and the block meets at its barriers half as often.
template <int NPW, int MTL, int WARPS>
__global__ void __launch_bounds__(WARPS * MTL * 32)
latent_attention_mma_kernel(const float* __restrict__ qa, const __nv_bfloat16* __restrict__ cache,
                            const float* __restrict__ sink, const __nv_bfloat16* __restrict__ gate, int ldg,
                            __nv_bfloat16* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml,
                            int num_splits, const int* __restrict__ cu_q, const int* __restrict__ pos0,
                            const int* __restrict__ entry_of_token, const int* __restrict__ block_table,
                            int bt_stride, int entry0, int H, int R, int r, int page_size, int num_pages, int window,
                            float scale, int hpb, int* status) {
  ccb::pdl_begin();
  constexpr int ROWS = 16 * MTL, KEYS = 8 * WARPS, LDP = KEYS + 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int W = R + r, LDW = W + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);              // [ROWS][LDW]
  __nv_bfloat16* Ct = Qs + ROWS * LDW;                                          // [2][KEYS][LDW]
  __nv_bfloat16* Ps = Ct + 2 * KEYS * LDW;                                  // [ROWS][LDP]
  float* red_max = reinterpret_cast<float*>(Ps + ROWS * LDP + 32);               // [4][ROWS] (after 64 bytes of slack)
  float* red_sum = red_max + WARPS * ROWS;                                  // [4][ROWS]
  const int tq = ROWS / hpb;
  const int e = entry0 + blockIdx.z / num_splits, split = blockIdx.z % num_splits;
  const int r0 = cu_q[e], n = cu_q[e + 1] - r0;
  const int qbase = blockIdx.x * tq;
  if (qbase >= n || entry_of_token[r0 + qbase] < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  constexpr int NW = WARPS * MTL;
  const int wk = warp % WARPS, rt0 = warp / WARPS;
  const int nq = min(tq, n - qbase);
  const int p_first = pos0[e] + qbase, p_last = p_first + nq - 1;
  const int j_lo = max(0, p_first - window + 1);
  const int* bt = block_table + (size_t)e * bt_stride;
  const int h0 = blockIdx.y * hpb;

  // this thread's rows, two in every tile of 16: (query, head), whether they exist, their position
  int row_t[1][2], row_h[1][2], row_p[1][2];
  bool row_ok[1][2];
#pragma unroll
  for (int rt = 0; rt < 1; ++rt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int rr = 16 * (rt0 + rt) + gid + 8 * hh, qi = rr / hpb, hd = h0 + rr % hpb;
      row_ok[rt][hh] = rr < tq * hpb && qi < nq && hd < H;
      row_t[rt][hh] = r0 + qbase + qi;
      row_h[rt][hh] = hd;
      row_p[rt][hh] = p_first + qi;
    }
  for (int i = threadIdx.x; i < ROWS * W; i += NW * 32) {
    const int rr = i / W, c = i - rr * W, qi = rr / hpb, hd = h0 + rr % hpb;
    const bool ok = rr < tq * hpb && qi < nq && hd < H;
    Qs[rr * LDW + c] = __float2bfloat16_rn(ok ? qa[((size_t)(r0 + qbase + qi) * H + hd) * W + c] : 0.f);
  }

  const int tile0 = j_lo / KEYS, n_tiles = p_last / KEYS - tile0 + 1;
  const int per = (n_tiles + num_splits - 1) / num_splits;
  const int t_begin = tile0 + split * per, t_end = min(tile0 + n_tiles, t_begin + per);
  const int chunks = W >> 3;   // 16-byte pieces of a row
  auto fetch = [&](int tile, int buf) {   // a warp takes every fourth row; its page is looked up once
    __nv_bfloat16* dst = Ct + (size_t)buf * KEYS * LDW;
#pragma unroll 2
    for (int rr = warp; rr < KEYS; rr += NW) {
      const int j = tile * KEYS + rr;
      const __nv_bfloat16* src = cache;
      bool ok = j >= j_lo && j <= p_last;
      if (ok) {
        const int lp = j / page_size;
        const int page = lp < bt_stride ? bt[lp] : -1;
        if (page < 0 || page >= num_pages) {
          if (lane == 0) set_status(status, CCB_ST_BAD_PAGE);
          ok = false;
        } else {
          src = cache + ((size_t)page * page_size + (j - lp * page_size)) * W;
        }
      }
      const uint32_t d = smem_u32(dst + rr * LDW);
      for (int c = lane; c < chunks; c += 32) cp_async16(d + c * 16, src + (ok ? c * 8 : 0), ok);
    }
    cp_async_commit();
  };

  float m[1][2], l[1][2], acc[1][NPW][2][4];
#pragma unroll
  for (int rt = 0; rt < 1; ++rt) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const bool first = split == 0 && row_ok[rt][hh];   // the sink: one term exp(sink) with no key and no value
      m[rt][hh] = first ? sink[row_h[rt][hh]] : -CUDART_INF_F;
      l[rt][hh] = first ? 1.f : 0.f;
    }
#pragma unroll
    for (int i = 0; i < NPW; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[rt][i][j][k] = 0.f;
  }

  const int n_pairs = R >> 4;
  if (t_begin < t_end) fetch(t_begin, 0);
  for (int tile = t_begin; tile < t_end; ++tile) {
    const int buf = (tile - t_begin) & 1;
    if (tile + 1 < t_end) {
      fetch(tile + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();   // the tile (and, the first time, Q) is in shared memory for everyone
    const __nv_bfloat16* C = Ct + (size_t)buf * KEYS * LDW;
    // ---- S = Q C^T for this warp's 8 keys (two chains of products per tile of rows)
    float sc[1][4], sc_odd[1][4];
#pragma unroll
    for (int rt = 0; rt < 1; ++rt)
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[rt][i] = sc_odd[rt][i] = 0.f;
    const uint32_t q_addr = smem_u32(Qs + (lane & 15) * LDW + (lane >> 4) * 8);
    const uint32_t k_addr = smem_u32(C + (8 * wk + (lane & 7)) * LDW + (lane >> 3) * 8);
    const int ksteps = W >> 4;
#pragma unroll 3
    for (int ks = 0; ks < ksteps; ks += 2) {
      uint32_t b[4];
      ldmatrix_x4(b[0], b[1], b[2], b[3], k_addr + ks * 32);
      const bool two = ks + 1 < ksteps;
#pragma unroll
      for (int rt = 0; rt < 1; ++rt) {
        uint32_t a[4], a2[4];
        ldmatrix_x4(a[0], a[1], a[2], a[3], q_addr + ((rt0 + rt) * 16 * LDW) * 2 + ks * 32);
        if (two) ldmatrix_x4(a2[0], a2[1], a2[2], a2[3], q_addr + ((rt0 + rt) * 16 * LDW) * 2 + (ks + 1) * 32);
        mma_bf16_16816(sc[rt], a, b[0], b[1]);
        if (two) mma_bf16_16816(sc_odd[rt], a2, b[2], b[3]);
      }
    }
    // ---- softmax over the staged keys
    const int jk = tile * KEYS + 8 * wk + 2 * tig;
#pragma unroll
    for (int rt = 0; rt < 1; ++rt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int lo = max(0, row_p[rt][hh] - window + 1);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int j = jk + c;
          const bool seen = row_ok[rt][hh] && j >= lo && j <= row_p[rt][hh];
          sc[rt][2 * hh + c] = seen ? (sc[rt][2 * hh + c] + sc_odd[rt][2 * hh + c]) * scale : -CUDART_INF_F;
        }
        float v = fmaxf(sc[rt][2 * hh], sc[rt][2 * hh + 1]);
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
        if (tig == 0) red_max[wk * ROWS + 16 * (rt0 + rt) + gid + 8 * hh] = v;
      }
    __syncthreads();
    float corr[1][2];
#pragma unroll
    for (int rt = 0; rt < 1; ++rt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int rr = 16 * (rt0 + rt) + gid + 8 * hh;
        float mn = m[rt][hh];
#pragma unroll
        for (int w = 0; w < WARPS; ++w) mn = fmaxf(mn, red_max[w * ROWS + rr]);
        const bool none = mn == -CUDART_INF_F;   // nothing seen so far (a piece without the sink)
        corr[rt][hh] = none ? 1.f : expf(m[rt][hh] - mn);
        m[rt][hh] = mn;
        const float p0 = none ? 0.f : expf(sc[rt][2 * hh] - mn), p1 = none ? 0.f : expf(sc[rt][2 * hh + 1] - mn);
        float ps = p0 + p1;
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        if (tig == 0) red_sum[wk * ROWS + rr] = ps;
        *reinterpret_cast<uint32_t*>(Ps + rr * LDP + 8 * wk + 2 * tig) = pack_bf16(p0, p1);
      }
    __syncthreads();
    uint32_t pa[1][KEYS / 16][4];
    const uint32_t p_addr = smem_u32(Ps + (lane & 15) * LDP + (lane >> 4) * 8);
#pragma unroll
    for (int rt = 0; rt < 1; ++rt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int rr = 16 * (rt0 + rt) + gid + 8 * hh;
        float ps = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) ps += red_sum[w * ROWS + rr];
        l[rt][hh] = l[rt][hh] * corr[rt][hh] + ps;
      }
#pragma unroll
      for (int ks = 0; ks < KEYS / 16; ++ks)
        ldmatrix_x4(pa[rt][ks][0], pa[rt][ks][1], pa[rt][ks][2], pa[rt][ks][3], p_addr + (rt0 + rt) * 16 * LDP * 2 + ks * 32);
    }
    // ---- O += P C for this warp's columns
    const uint32_t v_addr = smem_u32(C + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDW + (lane >> 4) * 8);
#pragma unroll
    for (int i = 0; i < NPW; ++i) {
      const int np = wk + WARPS * i;
      if (np < n_pairs) {
#pragma unroll
        for (int rt = 0; rt < 1; ++rt)
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            acc[rt][i][j][0] *= corr[rt][0]; acc[rt][i][j][1] *= corr[rt][0];
            acc[rt][i][j][2] *= corr[rt][1]; acc[rt][i][j][3] *= corr[rt][1];
          }
#pragma unroll
        for (int ks = 0; ks < KEYS / 16; ++ks) {
          uint32_t b[4];
          ldmatrix_x4_trans(b[0], b[1], b[2], b[3], v_addr + (ks * 16 * LDW + np * 16) * 2);
#pragma unroll
          for (int rt = 0; rt < 1; ++rt) {
            mma_bf16_16816(acc[rt][i][0], pa[rt][ks], b[0], b[1]);
            mma_bf16_16816(acc[rt][i][1], pa[rt][ks], b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();   // everyone is done with this buffer, P and the exchange arrays
  }
  // ---- the rows leave: finished (one piece) or as a piece of a row
#pragma unroll
  for (int rt = 0; rt < 1; ++rt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      if (!row_ok[rt][hh]) continue;
      const size_t row = (size_t)row_t[rt][hh] * H + row_h[rt][hh];
      if (num_splits == 1) {
        const float g = gate ? 1.0f / (1.0f + expf(-to_f32(gate[(size_t)row_t[rt][hh] * ldg + row_h[rt][hh]]))) : 1.0f;
        const float f = g / l[rt][hh];
#pragma unroll
        for (int i = 0; i < NPW; ++i) {
          const int np = wk + WARPS * i;
          if (np < n_pairs)
#pragma unroll
            for (int j = 0; j < 2; ++j)
              *reinterpret_cast<uint32_t*>(out + row * R + np * 16 + j * 8 + 2 * tig) =
                  pack_bf16(acc[rt][i][j][2 * hh] * f, acc[rt][i][j][2 * hh + 1] * f);
        }
      } else {
        float* pa_out = part_acc + (row * num_splits + split) * R;
#pragma unroll
        for (int i = 0; i < NPW; ++i) {
          const int np = wk + WARPS * i;
          if (np < n_pairs)
#pragma unroll
            for (int j = 0; j < 2; ++j)
              *reinterpret_cast<float2*>(pa_out + np * 16 + j * 8 + 2 * tig) =
                  make_float2(acc[rt][i][j][2 * hh], acc[rt][i][j][2 * hh + 1]);
        }
        if (wk == 0 && tig == 0) {
          part_ml[(row * num_splits + split) * 2] = m[rt][hh];
          part_ml[(row * num_splits + split) * 2 + 1] = l[rt][hh];
        }
      }
    }
}

// out[t, h, :] = sigmoid(gate) * sum_s acc_s exp(m_s - M) / sum_s l_s exp(m_s - M); a block per (token, head),
// a thread per column; the pieces' factors are worked out once, by the first warp
constexpr int kMergeThreads = 128;
constexpr int kMergeMaxSplits = 64;

__global__ void __launch_bounds__(kMergeThreads)
latent_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, int num_splits,
                    const __nv_bfloat16* __restrict__ gate, int ldg, __nv_bfloat16* __restrict__ out,
                    const int* __restrict__ entry_of_token, int row_begin, int H, int R) {
  ccb::pdl_begin();
  __shared__ float f[kMergeMaxSplits];
  const int t = row_begin + blockIdx.x / H, h = blockIdx.x % H;
  if (entry_of_token[t] < 0) return;
  const size_t row = (size_t)t * H + h;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float ms[2], ls[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int s = lane + 32 * i;
      ms[i] = s < num_splits ? part_ml[(row * num_splits + s) * 2] : -CUDART_INF_F;
      ls[i] = s < num_splits ? part_ml[(row * num_splits + s) * 2 + 1] : 0.f;
    }
    const float M = warp_max(fmaxf(ms[0], ms[1]));   // finite: piece 0 holds the sink
    float e[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) e[i] = ms[i] == -CUDART_INF_F ? 0.f : expf(ms[i] - M);
    const float L = warp_sum(ls[0] * e[0] + ls[1] * e[1]);
    const float g = gate ? 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * ldg + h]))) : 1.0f;
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (lane + 32 * i < num_splits) f[lane + 32 * i] = e[i] * g / L;
  }
  __syncthreads();
  const float* pa = part_acc + row * num_splits * R;
  const int c = blockIdx.y * kMergeThreads + threadIdx.x;   // a column a thread
  if (c < R) {
    float v0 = 0.f, v1 = 0.f;
    int s = 0;
    for (; s + 1 < num_splits; s += 2) {
      v0 = fmaf(pa[(size_t)s * R + c], f[s], v0);
      v1 = fmaf(pa[(size_t)(s + 1) * R + c], f[s + 1], v1);
    }
    if (s < num_splits) v0 = fmaf(pa[(size_t)s * R + c], f[s], v0);
    out[row * R + c] = __float2bfloat16_rn(v0 + v1);
  }
}

template <typename T, int NV>
int launch_attention(const float* qa, const void* cache, const float* sink, const void* gate, int ldg, void* out,
                     const int* cu_q, const int* pos0, const int* eot, const int* block_table, int bt_stride, int entry0, int n_entries,
                     int max_q, int H, int R, int r, int page_size, int num_pages, int window, float scale,
                     int* status, cudaStream_t stream) {
  // a block's warps share the staged rows: first among the heads of one query (they see the same keys), and
  // where a layer has fewer heads than a block has warps, among neighbouring queries too
  int hg = 1;
  while (hg < kAttWarps && hg < H) hg *= 2;
  const int tq = kAttWarps / hg;
  const int W = R + r;
  const size_t smem = ((size_t)kKeys * (W | 1) + (size_t)kAttWarps * W) * sizeof(float);
  if (smem > 200 * 1024) return CCB_REFUSE_SIZE;
  cudaFuncSetAttribute(latent_attention_kernel<T, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid((max_q + tq - 1) / tq, (H + hg - 1) / hg, n_entries);
  ccb_launch(latent_attention_kernel<T, NV>, grid, dim3(kAttWarps * 32), smem, stream, qa, (const T*)cache, sink,
             (const T*)gate, ldg, (T*)out, cu_q, pos0, eot, block_table, bt_stride, entry0, H, R, r, page_size,
             num_pages, window, scale, tq, status);
  return ccb_launch_status();
}

template <typename T>
int pick_attention(const float* qa, const void* cache, const float* sink, const void* gate, int ldg, void* out,
                   const int* cu_q, const int* pos0, const int* eot, const int* block_table, int bt_stride, int entry0, int n_entries,
                   int max_q, int H, int R, int r, int page_size, int num_pages, int window, float scale, int* status,
                   cudaStream_t stream) {
#define CCB_LAT(NV)                                                                                              \
  return launch_attention<T, NV>(qa, cache, sink, gate, ldg, out, cu_q, pos0, eot, block_table, bt_stride, entry0, \
                                 n_entries, max_q, H, R, r, page_size, num_pages, window, scale, status, stream)
  if (R <= 32) CCB_LAT(1);
  if (R <= 64) CCB_LAT(2);
  if (R <= 128) CCB_LAT(4);
  if (R <= 256) CCB_LAT(8);
  if (R <= 512) CCB_LAT(16);
  if (R <= 1024) CCB_LAT(32);
#undef CCB_LAT
  return CCB_REFUSE_SIZE;
}

}  // namespace

CCB_API int ccb_latent_prepare(const void* proj, int ld, int oq, int oc, const float* w, const float* inv_freq,
                               int rot_dims, const int* positions, const int* slot_map, void* cache, int num_slots,
                               float* qa, int T, int H, int d, int r, int R, float eps, int dtype, int* status,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || d < 0 || r < 0 || R <= 0 || rot_dims < 0 || rot_dims > r || (rot_dims & 1)) return CCB_REFUSE_SIZE;
  if (rot_dims > 0 && inv_freq == nullptr) return CCB_REFUSE_ARG;
  // few tokens: a token's work is spread over several blocks (the cache row, and the heads' rotated parts in
  // pieces of about 512 coordinates)
  const int parts = T <= 64 ? 1 + min(8, (H * r + 511) / 512) : 1;
  const dim3 grid(T, parts);
  if (dtype == CCB_F32)
    ccb_launch(latent_prepare_kernel<float>, grid, dim3(kPrepThreads), 0, stream, (const float*)proj, ld, oq, oc, w,
               inv_freq, rot_dims, positions, slot_map, (float*)cache, num_slots, qa, H, d, r, R, eps, status);
  else if (dtype == CCB_BF16)
    ccb_launch(latent_prepare_kernel<__nv_bfloat16>, grid, dim3(kPrepThreads), 0, stream,
               (const __nv_bfloat16*)proj, ld, oq, oc, w, inv_freq, rot_dims, positions, slot_map,
               (__nv_bfloat16*)cache, num_slots, qa, H, d, r, R, eps, status);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// Entries entry0 .. entry0 + n_entries - 1 of the step, none with more than max_q tokens.
CCB_API int ccb_latent_attention(const float* qa, const void* cache, const float* sink, const void* gate, int ldg,
                                 void* out, const int* cu_q, const int* pos0, const int* entry_of_token,
                                 const int* block_table, int bt_stride, int entry0, int n_entries, int max_q, int H, int R, int r, int page_size,
                                 int num_pages, int window, float scale, int dtype, int* status,
                                 cudaStream_t stream) {
  if (n_entries <= 0 || max_q <= 0) return 0;
  if (H <= 0 || R <= 0 || r < 0 || page_size <= 0 || window <= 0 || n_entries > 65535) return CCB_REFUSE_SIZE;
  if (dtype == CCB_F32)
    return pick_attention<float>(qa, cache, sink, gate, ldg, out, cu_q, pos0, entry_of_token, block_table, bt_stride, entry0,
                                 n_entries, max_q, H, R, r, page_size, num_pages, window, scale, status, stream);
  if (dtype == CCB_BF16)
    return pick_attention<__nv_bfloat16>(qa, cache, sink, gate, ldg, out, cu_q, pos0, entry_of_token, block_table, bt_stride, entry0,
                                         n_entries, max_q, H, R, r, page_size, num_pages, window, scale, status,
                                         stream);
  return CCB_REFUSE_DTYPE;
}

namespace {
template <int NPW, int MTL, int WARPS>
int launch_mma(const float* qa, const void* cache, const float* sink, const void* gate, int ldg, void* out,
               float* part_acc, float* part_ml, int num_splits, const int* cu_q, const int* pos0, const int* eot,
               const int* block_table, int bt_stride, int entry0, int n_entries, int max_q, int H, int R, int r,
               int page_size, int num_pages, int window, float scale, int* status, cudaStream_t stream) {
  constexpr int ROWS = 16 * MTL, KEYS = 8 * WARPS;
  int hpb = 1;
  while (hpb < 16 && hpb < H) hpb *= 2;   // (with two tiles of rows a block still holds 16 heads at most)
  const int tq = ROWS / hpb;
  const int W = R + r;
  const size_t smem = (size_t)(ROWS + 2 * KEYS) * (W + 8) * 2 + ROWS * (KEYS + 8) * 2 + 64 + 2 * WARPS * ROWS * 4 + 64;
  cudaFuncSetAttribute(latent_attention_mma_kernel<NPW, MTL, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       (int)smem);
  dim3 grid((max_q + tq - 1) / tq, (H + hpb - 1) / hpb, n_entries * num_splits);
  ccb_launch(latent_attention_mma_kernel<NPW, MTL, WARPS>, grid, dim3(WARPS * MTL * 32), smem, stream, qa,
             (const __nv_bfloat16*)cache, sink, (const __nv_bfloat16*)gate, ldg, (__nv_bfloat16*)out, part_acc,
             part_ml, num_splits, cu_q, pos0, eot, block_table, bt_stride, entry0, H, R, r, page_size, num_pages,
             window, scale, hpb, status);
  return ccb_launch_status();
}
}  // namespace

// Whether the tensor-core form takes these sizes (bfloat16 only).
CCB_API int ccb_latent_attention_mma_fits(int R, int r) {
  return (R > 0 && R % 16 == 0 && r >= 0 && r % 16 == 0 && R <= 512) ? 1 : 0;
}

// As ccb_latent_attention, bfloat16, for single-token entries with `num_splits` > 1: entries entry0 .. are the
// token rows entry0 .. (a step lists its single tokens first), part_acc [rows * H * num_splits * R] and part_ml
// [rows * H * num_splits * 2] are float scratch.
CCB_API int ccb_latent_attention_mma(const float* qa, const void* cache, const float* sink, const void* gate, int ldg,
                                     void* out, float* part_acc, float* part_ml, int num_splits, const int* cu_q,
                                     const int* pos0, const int* entry_of_token, const int* block_table,
                                     int bt_stride, int entry0, int n_entries, int max_q, int H, int R, int r,
                                     int page_size, int num_pages, int window, float scale, int* status,
                                     cudaStream_t stream) {
  if (n_entries <= 0 || max_q <= 0) return 0;
  if (!ccb_latent_attention_mma_fits(R, r) || H <= 0 || page_size <= 0 || window <= 0 || num_splits < 1 ||
      (long long)n_entries * num_splits > 65535 || num_splits > kMergeMaxSplits || (num_splits > 1 && (max_q != 1 || !part_acc || !part_ml)))
    return CCB_REFUSE_SIZE;
  // portions of prompts: 32 (query, head) rows and 16 warps a block; single tokens: 16 rows and 4 warps
  const bool wide = max_q >= 16;
  const int warps = wide ? 8 : kMmaWarps;
  const int pairs_per_warp = ((R >> 4) + warps - 1) / warps;
  int rc;
#define CCB_LMMA(NPW, MTL, WARPS)                                                                                  \
  rc = launch_mma<NPW, MTL, WARPS>(qa, cache, sink, gate, ldg, out, part_acc, part_ml, num_splits, cu_q, pos0,     \
                                   entry_of_token, block_table, bt_stride, entry0, n_entries, max_q, H, R, r,      \
                                   page_size, num_pages, window, scale, status, stream)
  if (wide) {
    if (pairs_per_warp <= 1) CCB_LMMA(1, 2, 8);
    else if (pairs_per_warp <= 2) CCB_LMMA(2, 2, 8);
    else CCB_LMMA(4, 2, 8);
  } else {
    if (pairs_per_warp <= 1) CCB_LMMA(1, 1, 4);
    else if (pairs_per_warp <= 2) CCB_LMMA(2, 1, 4);
    else if (pairs_per_warp <= 4) CCB_LMMA(4, 1, 4);
    else CCB_LMMA(8, 1, 4);
  }
#undef CCB_LMMA
  if (rc != 0 || num_splits == 1) return rc;
  ccb_launch(latent_merge_kernel, dim3(n_entries * H, (R + kMergeThreads - 1) / kMergeThreads), dim3(kMergeThreads), 0, stream, part_acc, part_ml, num_splits,
             (const __nv_bfloat16*)gate, ldg, (__nv_bfloat16*)out, entry_of_token, entry0, H, R);
  return ccb_launch_status();
}
