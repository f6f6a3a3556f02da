// The grouped products of a mixture of experts on the 5th-generation tensor cores, for steps in which an expert
// gets many rows: C[row, :] = A[row, :] W_e^T for the rows of every tile of 128 sorted rows, W_e the tile's expert.
//
// It is the tcgen05 product of gemm_tcgen05.cu (TMA loads with 128-byte swizzle, one thread issuing tcgen05.mma
// with the accumulator in tensor memory, four epilogue warps reading it back) with three differences:
//   * a block takes its rows from the tile list of moe_sort (first sorted row, number of rows, expert) instead
//     of from its place in the grid; rows of the 128 beyond the tile's own belong to the next expert and are
//     computed but not stored;
//   * the weight operand is ONE tensor map over all experts' matrices, and the expert moves the box: down the
//     rows (the first matrices, stacked [E F, D]) or along the columns (the second ones, side by side [D, E F];
//     what a box reads beyond the expert's F columns meets zeros of A, whose map ends at F);
//   * the epilogue of the first product is relu(c)^2 * weight(row) in bfloat16, that of the second float.
// The rows of A must lie in sorted order, so the tokens are gathered first (moe_gather_rows).
// Every wait on an mbarrier is bounded as in gemm_tcgen05.cu.
#include "common.cuh"
#include <cuda.h>

#include "tc_common.cuh"
#include "tma_host.h"

using namespace ccb;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int kThreadsTc = 192;

__host__ __device__ constexpr uint32_t instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// MODE 0: B rows at e * F + tile column, C bfloat16 = relu(c)^2 * row_w;  MODE 1: B columns at e * F + k, C float;
// MODE 2: as MODE 0 with B's rows gate and up rows in turn (F rows an expert, N = F), C bfloat16 [*, N / 2] =
// silu(gate) * up * row_w.
template <int BN, int STAGES, int MODE>
__global__ void __launch_bounds__(kThreadsTc, 1)
moe_grouped_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      void* __restrict__ Cout, int ldc, const float* __restrict__ row_w,
                      const int* __restrict__ tile_e, const int* __restrict__ tile_r0,
                      const int* __restrict__ tile_n, int N, int K, int F, int* status) {
  ccb::pdl_begin();
  const int n_rows = tile_n[blockIdx.x];
  if (n_rows <= 0) return;   // (the whole block, before anything is set up)
  const int e = tile_e[blockIdx.x], r0 = tile_r0[blockIdx.x];
  constexpr int B_STAGE_BYTES = BN * BK * 2;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + STAGES * B_STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  const uint32_t full0 = s32(bars), empty0 = s32(bars + STAGES), tfull = s32(bars + 2 * STAGES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tileB = blockIdx.y;
  const int nkb = (K + BK - 1) / BK;
  const int b_row = MODE != 1 ? e * F + tileB * BN : tileB * BN;
  const int b_col = MODE != 1 ? 0 : e * F;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(tfull, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer ----
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES, ph = (i / STAGES) & 1;
        if (i >= STAGES && !mbar_wait(empty0 + 8 * s, ph ^ 1)) {
          set_status(status, CCB_ST_WAIT_TIMEOUT);
          break;
        }
        mbar_expect_tx(full0 + 8 * s, A_STAGE_BYTES + B_STAGE_BYTES);
        tma_load_2d(s32(sA + s * A_STAGE_BYTES), &tmA, i * BK, r0, full0 + 8 * s);
        tma_load_2d(s32(sB + s * B_STAGE_BYTES), &tmB, b_col + i * BK, b_row, full0 + 8 * s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer ----
      constexpr uint32_t idesc = instr_desc(BN);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES, ph = (i / STAGES) & 1;
        if (!mbar_wait(full0 + 8 * s, ph)) {
          set_status(status, CCB_ST_WAIT_TIMEOUT);
          break;
        }
        tc_fence_after();
        const uint64_t da = smem_desc(s32(sA + s * A_STAGE_BYTES));
        const uint64_t db = smem_desc(s32(sB + s * B_STAGE_BYTES));
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          tc_mma(tmem_base, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        tc_commit(empty0 + 8 * s);
      }
      tc_commit(tfull);
    }
  } else {  // ---- epilogue: warp q reads TMEM lanes 32 q .. 32 q + 31 ----
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool ok = mbar_wait(tfull, 0);
    if (!ok && lane == 0) set_status(status, CCB_ST_WAIT_TIMEOUT);
    tc_fence_after();
    if (ok) {
      const size_t g = (size_t)(r0 + row);
      const bool mine = row < n_rows;
      const float wr = (MODE != 1 && mine) ? row_w[g] : 1.f;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t v[16];
        tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + c0, v);
        tc_wait_ld();
        const int col = tileB * BN + c0;
        const int n_valid = min(16, N - col);
        if (!mine || n_valid <= 0) continue;
        if (MODE == 0) {
          __nv_bfloat16* dst = (__nv_bfloat16*)Cout + g * ldc + col;
          uint32_t p[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float a = fmaxf(__uint_as_float(v[2 * i]), 0.f), b = fmaxf(__uint_as_float(v[2 * i + 1]), 0.f);
            const __nv_bfloat162 h = __floats2bfloat162_rn(a * a * wr, b * b * wr);
            p[i] = *reinterpret_cast<const uint32_t*>(&h);
          }
          if (n_valid == 16 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(p[0], p[1], p[2], p[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(p[4], p[5], p[6], p[7]);
          } else {
            const __nv_bfloat16* ph = reinterpret_cast<const __nv_bfloat16*>(p);
            for (int i = 0; i < n_valid; ++i) dst[i] = ph[i];
          }
        } else if (MODE == 2) {   // columns (2 f, 2 f + 1) are gate f and up f
          __nv_bfloat16* dst = (__nv_bfloat16*)Cout + g * ldc + (col >> 1);
          uint32_t p[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float g0 = __uint_as_float(v[4 * i]), u0 = __uint_as_float(v[4 * i + 1]);
            const float g1 = __uint_as_float(v[4 * i + 2]), u1 = __uint_as_float(v[4 * i + 3]);
            const __nv_bfloat162 h = __floats2bfloat162_rn(g0 / (1.f + __expf(-g0)) * u0 * wr,
                                                           g1 / (1.f + __expf(-g1)) * u1 * wr);
            p[i] = *reinterpret_cast<const uint32_t*>(&h);
          }
          if (n_valid == 16 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(p[0], p[1], p[2], p[3]);
          } else {
            const __nv_bfloat16* ph = reinterpret_cast<const __nv_bfloat16*>(p);
            for (int i = 0; i < n_valid / 2; ++i) dst[i] = ph[i];
          }
        } else {
          float* dst = (float*)Cout + g * ldc + col;
          if (n_valid == 16 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              reinterpret_cast<uint4*>(dst)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          } else {
            for (int i = 0; i < n_valid; ++i) dst[i] = __uint_as_float(v[i]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

// out[pos, :] = x[src_row[pos], :]: the tokens in sorted order, 16 bytes a thread and step
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(uint4* __restrict__ out, const uint4* __restrict__ x, const int* __restrict__ src_row, int ldx16,
                       int row16, size_t total) {
  ccb::pdl_begin();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t pos = i / row16;
    const int c = (int)(i - pos * row16);
    out[i] = x[(size_t)src_row[pos] * ldx16 + c];
  }
}

template <int MODE>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, void* C, int ldc, const float* row_w, const int* tile_e,
           const int* tile_r0, const int* tile_n, int max_tiles, int N, int K, int F, int* status,
           cudaStream_t stream) {
  constexpr int BN = 256, STAGES = 4;
  constexpr size_t smem = (size_t)STAGES * (A_STAGE_BYTES + BN * BK * 2) + (2 * STAGES + 1) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_grouped_tc_kernel<BN, STAGES, MODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  ccb_launch(moe_grouped_tc_kernel<BN, STAGES, MODE>, dim3(max_tiles, (N + BN - 1) / BN), dim3(kThreadsTc), smem,
             stream, tmA, tmB, C, ldc, row_w, tile_e, tile_r0, tile_n, N, K, F, status);
  return ccb_launch_status();
}

}  // namespace

// bfloat16 rows of `width` elements (a multiple of 8), x rows at ldx: out [rows, width] = x[src_row[.]]
CCB_API int ccb_moe_gather_rows(void* out, const void* x, const int* src_row, int rows, int width, int ldx,
                                cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (width <= 0 || (width & 7) || (ldx & 7) || (reinterpret_cast<uintptr_t>(out) & 15) ||
      (reinterpret_cast<uintptr_t>(x) & 15))
    return CCB_REFUSE_SIZE;
  const size_t total = (size_t)rows * (width / 8);
  const int blocks = (int)((total + 255) / 256 < 65535 * 8 ? (total + 255) / 256 : 65535 * 8);
  ccb_launch(moe_gather_rows_kernel, dim3(blocks), dim3(256), 0, stream, (uint4*)out, (const uint4*)x, src_row, ldx / 8,
             width / 8, total);
  return ccb_launch_status();
}

// The tiles are those of moe_sort with BM = 128.  A [rows, K] holds the sorted rows (contiguous rows of lda).
// mode 0: W = the first matrices stacked [w_rows, K] (expert e at row e * F), C bfloat16 [rows, N = F] with
// relu(.)^2 * row_w;  mode 1: W = the second matrices side by side [N, w_cols] (expert e at column e * F, K = F),
// C float [rows, N];  mode 2: W = the first matrices stacked with every expert's gate and up rows in turn (F rows an
// expert, N = F), C bfloat16 [rows, N / 2] = silu(gate) * up * row_w.
CCB_API int ccb_moe_grouped_tc(const void* A, int lda, int rows, const void* W, int ldw, int w_rows, int w_cols,
                               void* C, int ldc, const float* row_w, const int* tile_e, const int* tile_r0,
                               const int* tile_n, int max_tiles, int N, int K, int F, int mode, int* status,
                               cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0 || rows <= 0) return 0;
  if (K <= 0 || (K & 7) || (F & 7) || (lda & 7) || (ldw & 7) || mode < 0 || mode > 2 || (mode == 2 && (N & 1)) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return CCB_REFUSE_SIZE;
  CUtensorMap tmA, tmB;
  if (!ccb_tensor_map_2d(A, rows, K, lda, BK, BM, &tmA) || !ccb_tensor_map_2d(W, w_rows, w_cols, ldw, BK, 256, &tmB))
    return CCB_REFUSE_ARG;
  if (mode == 2)
    return launch<2>(tmA, tmB, C, ldc, row_w, tile_e, tile_r0, tile_n, max_tiles, N, K, F, status, stream);
  if (mode == 0)
    return launch<0>(tmA, tmB, C, ldc, row_w, tile_e, tile_r0, tile_n, max_tiles, N, K, F, status, stream);
  return launch<1>(tmA, tmB, C, ldc, row_w, tile_e, tile_r0, tile_n, max_tiles, N, K, F, status, stream);
}
