// Host-side tensor maps for TMA (cuTensorMapEncodeTiled through the runtime's driver entry point); see tma_host.h.
// Every kernel family links this file and keeps its own cache of maps.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <map>
#include <mutex>
#include <tuple>

#include "tma_host.h"

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}


// tensor maps are cached by (pointer, rows, columns, row stride, box, swizzle): weights and the engine's scratch
// buffers keep their addresses for the life of the process
static std::mutex g_mu;
static std::map<std::tuple<const void*, unsigned long long, unsigned long long, unsigned long long, unsigned, unsigned, int>,
                CUtensorMap> g_maps;

static bool tensor_map_2d(const void* ptr, unsigned long long rows, unsigned long long cols, unsigned long long ld,
                          unsigned box_cols, unsigned box_rows, bool swizzle128, CUtensorMap* out) {
  const auto key = std::make_tuple(ptr, rows, cols, ld, box_cols, box_rows, swizzle128 ? 1 : 0);
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return true;
  }
  auto fn = encode_fn();
  if (fn == nullptr) return false;
  CUtensorMap tm;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps[key] = tm;
  *out = tm;
  return true;
}

bool ccb_tensor_map_2d(const void* ptr, unsigned long long rows, unsigned long long cols, unsigned long long ld,
                       unsigned box_cols, unsigned box_rows, CUtensorMap* out) {
  return tensor_map_2d(ptr, rows, cols, ld, box_cols, box_rows, true, out);
}

bool ccb_tensor_map_2d_plain(const void* ptr, unsigned long long rows, unsigned long long cols, unsigned long long ld,
                             unsigned box_cols, unsigned box_rows, CUtensorMap* out) {
  return tensor_map_2d(ptr, rows, cols, ld, box_cols, box_rows, false, out);
}

