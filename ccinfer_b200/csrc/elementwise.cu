// Embedding gather and SiLU-multiply.
//
// embed:    h[t, :] = float(table[ids[t], :])          (7QiC/ccInfer: src/kernel/elementwise/elementwise.cu:67-78)
// silu_mul: act[t, f] = silu(gu[t, f]) * gu[t, F + f]  (7QiC/ccInfer: src/kernel/mlp/silu_mul.cu:24-28)
// The gate and up projections are one merged matrix product here, so the
// kernel reads both halves of a [T, 2F] row.
#include "common.cuh"

using namespace ccb;

template <typename T>
__global__ void embed_gather_kernel(float* __restrict__ h, const T* __restrict__ table,
                                    const int* __restrict__ ids, int D, int V, const int* __restrict__ pending,
                                    int n_pending, int* status) {
  ccb::pdl_begin();
  const int t = blockIdx.x;
  int id = ids[t];
  // id = -1 - s names the token that the sampling kernel last stored for request slot s: the host has
  // launched this step before it has read that token
  if (id < 0 && pending != nullptr && -1 - id < n_pending) id = pending[-1 - id];
  float* out = h + (size_t)t * D;
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) set_status(status, CCB_ST_BAD_TOKEN);
    for (int d = threadIdx.x; d < D; d += blockDim.x) out[d] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) out[d] = to_f32(row[d]);
}

CCB_API int ccb_embed_gather(float* h, const void* table, const int* ids, int T_, int D, int V,
                             int dtype, const int* pending, int n_pending, int* status, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (D <= 0 || V <= 0) return CCB_REFUSE_SIZE;
  const int threads = D >= 1024 ? 256 : 128;
  if (dtype == CCB_F32)
    ccb_launch(embed_gather_kernel<float>, T_, threads, 0, stream, h, (const float*)table, ids, D, V, pending, n_pending, status);
  else if (dtype == CCB_BF16)
    ccb_launch(embed_gather_kernel<__nv_bfloat16>, T_, threads, 0, stream, h, (const __nv_bfloat16*)table, ids, D, V, pending,
               n_pending, status);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// accurate variant for the 32-bit path, fast exponential for the bf16 path
template <typename T> __device__ __forceinline__ float silu(float g);
template <> __device__ __forceinline__ float silu<float>(float g) { return g / (1.f + expf(-g)); }
template <> __device__ __forceinline__ float silu<__nv_bfloat16>(float g) { return g / (1.f + __expf(-g)); }

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ act, const T* __restrict__ gu, int F, int B, size_t total) {
  ccb::pdl_begin();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / F;
    const int f = (int)(i - t * F);
    const T* row = gu + t * 2 * (size_t)F;
    const int gi = (f / B) * 2 * B + f % B;  // B gate columns, then the B up columns of the same channels
    const float g = to_f32(row[gi]);
    const float u = to_f32(row[gi + B]);
    act[i] = from_f32<T>(silu<T>(g) * u);
  }
}

// bf16, F even: two elements per thread
__global__ void silu_mul_bf16x2_kernel(__nv_bfloat162* __restrict__ act, const __nv_bfloat162* __restrict__ gu,
                                       int F2, int B2, size_t total2) {
  ccb::pdl_begin();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total2; i += stride) {
    const size_t t = i / F2;
    const int f = (int)(i - t * F2);
    const __nv_bfloat162* row = gu + t * 2 * (size_t)F2;
    const int gi = (f / B2) * 2 * B2 + f % B2;
    const float2 g = __bfloat1622float2(row[gi]);
    const float2 u = __bfloat1622float2(row[gi + B2]);
    act[i] = __floats2bfloat162_rn(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
  }
}

// bf16, F a multiple of 8: eight elements (16 bytes) per thread and access
__global__ void silu_mul_bf16x8_kernel(uint4* __restrict__ act, const uint4* __restrict__ gu, int F8, int B8,
                                       size_t total8) {
  ccb::pdl_begin();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total8; i += stride) {
    const size_t t = i / F8;
    const int f = (int)(i - t * F8);
    const uint4* row = gu + t * 2 * (size_t)F8;
    const int gi = (f / B8) * 2 * B8 + f % B8;
    const uint4 g = row[gi], u = row[gi + B8];
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(gh[e]), b = __bfloat1622float2(uh[e]);
      oh[e] = __floats2bfloat162_rn(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
    }
    act[i] = o;
  }
}

// gate_up[t, :] holds the 2F columns either as [all gate | all up] (block = 0) or in blocks: `block` gate
// columns followed by the `block` up columns of the same channels (F a multiple of block).
CCB_API int ccb_silu_mul(void* act, const void* gate_up, int T_, int F, int block, int dtype, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (F <= 0 || block < 0 || (block > 0 && F % block != 0)) return CCB_REFUSE_SIZE;
  const int B = block == 0 ? F : block;
  const size_t total = (size_t)T_ * F;
  const int threads = 256;
  if (dtype == CCB_BF16 && (F % 8) == 0 && (B % 8) == 0 && ((reinterpret_cast<uintptr_t>(act) | reinterpret_cast<uintptr_t>(gate_up)) & 15) == 0) {
    const size_t total8 = total / 8;
    const size_t want = (total8 + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
    ccb_launch(silu_mul_bf16x8_kernel, blocks, threads, 0, stream, (uint4*)act, (const uint4*)gate_up, F / 8, B / 8,
               total8);
    return ccb_launch_status();
  }
  if (dtype == CCB_BF16 && (F % 2) == 0 && (B % 2) == 0) {
    const size_t total2 = total / 2;
    const int blocks = (int)((total2 + threads - 1) / threads < 148 * 16 ? (total2 + threads - 1) / threads : 148 * 16);
    ccb_launch(silu_mul_bf16x2_kernel, blocks, threads, 0, stream, (__nv_bfloat162*)act, (const __nv_bfloat162*)gate_up,
               F / 2, B / 2, total2);
    return ccb_launch_status();
  }
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == CCB_F32)
    ccb_launch(silu_mul_kernel<float>, blocks, threads, 0, stream, (float*)act, (const float*)gate_up, F, B, total);
  else if (dtype == CCB_BF16)
    ccb_launch(silu_mul_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16*)act, (const __nv_bfloat16*)gate_up, F, B,
               total);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// Gated activation with clamped inputs:
//   g = min(gate, limit), u = clamp(up, -limit, limit);  act = g * sigmoid(alpha * g) * (u + up_shift)
// over the same two layouts of the merged gate|up columns as silu_mul.  Arithmetic in float.
template <typename T>
__global__ void clamped_glu_kernel(T* __restrict__ act, const T* __restrict__ gu, int F, int B, size_t total,
                                   float limit, float alpha, float up_shift) {
  ccb::pdl_begin();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / F;
    const int f = (int)(i - t * F);
    const T* row = gu + t * 2 * (size_t)F;
    const int gi = (f / B) * 2 * B + f % B;
    const float g = fminf(to_f32(row[gi]), limit);
    const float u = fminf(fmaxf(to_f32(row[gi + B]), -limit), limit);
    act[i] = from_f32<T>(g / (1.0f + expf(-alpha * g)) * (u + up_shift));
  }
}

// bf16, F and the block multiples of 8: eight elements (16 bytes) per thread and access
__global__ void clamped_glu_bf16x8_kernel(uint4* __restrict__ act, const uint4* __restrict__ gu, int F8, int B8,
                                          size_t total8, const CcbGluAct a) {
  ccb::pdl_begin();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total8; i += stride) {
    const size_t t = i / F8;
    const int f = (int)(i - t * F8);
    const uint4* row = gu + t * 2 * (size_t)F8;
    const int gi = (f / B8) * 2 * B8 + f % B8;
    const uint4 g = row[gi], u = row[gi + B8];
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = __bfloat1622float2(gh[e]), y = __bfloat1622float2(uh[e]);
      oh[e] = __floats2bfloat162_rn(glu_act(a, x.x, y.x), glu_act(a, x.y, y.y));
    }
    act[i] = o;
  }
}

CCB_API int ccb_clamped_glu(void* act, const void* gate_up, int T_, int F, int block, float limit, float alpha,
                            float up_shift, int dtype, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (F <= 0 || block < 0 || (block > 0 && F % block != 0)) return CCB_REFUSE_SIZE;
  const int B = block == 0 ? F : block;
  const size_t total = (size_t)T_ * F;
  const int threads = 256;
  if (dtype == CCB_BF16 && limit > 0.f && (F % 8) == 0 && (B % 8) == 0 &&
      ((reinterpret_cast<uintptr_t>(act) | reinterpret_cast<uintptr_t>(gate_up)) & 15) == 0) {
    const size_t total8 = total / 8;
    const size_t want = (total8 + threads - 1) / threads;
    ccb_launch(clamped_glu_bf16x8_kernel, (int)(want < 148 * 32 ? want : 148 * 32), threads, 0, stream, (uint4*)act,
               (const uint4*)gate_up, F / 8, B / 8, total8, CcbGluAct{limit, alpha, up_shift});
    return ccb_launch_status();
  }
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == CCB_F32)
    ccb_launch(clamped_glu_kernel<float>, blocks, threads, 0, stream, (float*)act, (const float*)gate_up, F, B, total,
               limit, alpha, up_shift);
  else if (dtype == CCB_BF16)
    ccb_launch(clamped_glu_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16*)act,
               (const __nv_bfloat16*)gate_up, F, B, total, limit, alpha, up_shift);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// ---------------------------------------------------------------------------------------------
// out[t, :] = [a[t, :] | b[t, :]] in the storage type: two float streams side by side as the rows of a product.
template <typename T>
__global__ void concat_cast_kernel(T* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b,
                                   int D, size_t total) {
  ccb::pdl_begin();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / (2 * (size_t)D);
    const int c = (int)(i - t * 2 * D);
    out[i] = from_f32<T>(c < D ? a[t * D + c] : b[t * D + c - D]);
  }
}

// four columns a thread (D a multiple of 4, 16-byte bases)
template <typename T>
__global__ void concat_cast_vec_kernel(T* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b,
                                       int D, size_t total4) {
  ccb::pdl_begin();
  const int d4 = D >> 1;   // groups of four in a row of 2 D
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / d4;
    const int c = (int)(i - t * d4) * 4;
    const float4 v = *reinterpret_cast<const float4*>(c < D ? a + t * D + c : b + t * D + c - D);
    T* dst = out + t * 2 * (size_t)D + c;
    if constexpr (sizeof(T) == 4) {
      *reinterpret_cast<float4*>(dst) = v;
    } else {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
      uint2 r;
      r.x = *reinterpret_cast<const uint32_t*>(&lo);
      r.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(dst) = r;
    }
  }
}

CCB_API int ccb_concat_cast(void* out, const float* a, const float* b, int rows, int D, int dtype,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D <= 0) return CCB_REFUSE_SIZE;
  if (D % 4 == 0 && (dtype == CCB_F32 || dtype == CCB_BF16) &&
      ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0) {
    const size_t total4 = (size_t)rows * (D / 2);
    const int blocks4 = (int)((total4 + 255) / 256 < 65535 * 8 ? (total4 + 255) / 256 : 65535 * 8);
    if (dtype == CCB_F32)
      ccb_launch(concat_cast_vec_kernel<float>, dim3(blocks4), dim3(256), 0, stream, (float*)out, a, b, D, total4);
    else
      ccb_launch(concat_cast_vec_kernel<__nv_bfloat16>, dim3(blocks4), dim3(256), 0, stream, (__nv_bfloat16*)out, a, b,
                 D, total4);
    return ccb_launch_status();
  }
  const size_t total = (size_t)rows * 2 * D;
  const int blocks = (int)((total + 255) / 256 < 65535 * 8 ? (total + 255) / 256 : 65535 * 8);
  if (dtype == CCB_F32)
    ccb_launch(concat_cast_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)out, a, b, D, total);
  else if (dtype == CCB_BF16)
    ccb_launch(concat_cast_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)out, a, b, D, total);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// h[t, :] += row[:] (float): one vector added to every row of the stream.
__global__ void add_row_kernel(float* __restrict__ h, const float* __restrict__ row, int D, size_t total) {
  ccb::pdl_begin();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    h[i] += row[i % D];
}

CCB_API int ccb_add_row(float* h, const float* row, int rows, int D, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D <= 0) return CCB_REFUSE_SIZE;
  const size_t total = (size_t)rows * D;
  const int blocks = (int)((total + 255) / 256 < 65535 * 8 ? (total + 255) / 256 : 65535 * 8);
  ccb_launch(add_row_kernel, dim3(blocks), dim3(256), 0, stream, h, row, D, total);
  return ccb_launch_status();
}

// g[t, j] = gelu_tanh(g[t, j]) * table[ids[t], off + j], j < n: a gate times the token's own row of a second
// embedding table.  gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))), in float.
// Token ids as in embed_gather (-1 - s: the token last sampled for request slot s).
template <typename T>
__global__ void gelu_gate_rows_kernel(T* __restrict__ g, int ldg, const T* __restrict__ table, int ldt, int off,
                                      const int* __restrict__ ids, int n, int V, const int* __restrict__ pending,
                                      int n_pending, size_t total, int* status) {
  ccb::pdl_begin();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / n;
    const int j = (int)(i - t * n);
    int id = ids[t];
    if (id < 0 && pending != nullptr && -1 - id < n_pending) id = pending[-1 - id];
    T* p = g + t * ldg + j;
    if (id < 0 || id >= V) {
      set_status(status, CCB_ST_BAD_TOKEN);
      *p = from_f32<T>(0.f);
      continue;
    }
    const float z = to_f32(*p);
    const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    *p = from_f32<T>(0.5f * z * (1.f + tanhf(u)) * to_f32(table[(size_t)id * ldt + off + j]));
  }
}

CCB_API int ccb_gelu_gate_rows(void* g, int ldg, const void* table, int ldt, int off, const int* ids, int rows, int n,
                               int V, const int* pending, int n_pending, int dtype, int* status,
                               cudaStream_t stream) {
  if (rows <= 0 || n <= 0) return 0;
  if (V <= 0 || off < 0 || off + n > ldt || ldg < n) return CCB_REFUSE_SIZE;
  const size_t total = (size_t)rows * n;
  const int blocks = (int)((total + 255) / 256 < 65535 * 8 ? (total + 255) / 256 : 65535 * 8);
  if (dtype == CCB_F32)
    ccb_launch(gelu_gate_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)g, ldg, (const float*)table,
               ldt, off, ids, n, V, pending, n_pending, total, status);
  else if (dtype == CCB_BF16)
    ccb_launch(gelu_gate_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)g, ldg,
               (const __nv_bfloat16*)table, ldt, off, ids, n, V, pending, n_pending, total, status);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// ---------------------------------------------------------------------------------------------
// Token embedding times a constant, plus a row of a second table chosen by the pair (previous token, token):
//   h[t, :] = float(table[id, :]) * scale + float(pair_table[row, :])
//   row = (prev * mul_prev + id * mul_cur) mod buckets, or `buckets` (the table's last row) at position 0.
// The previous token of a portion's first token is what the request's slot of `prev_token` holds; the others find
// theirs in the step.  `rows` (optional): the same values in the storage type, for a block that reads the stream
// itself.  embed_pair_commit then stores each request's last token of the step (a kernel of its own: the first
// token's block of a request may run after the last one's).
template <typename T>
__global__ void embed_pair_kernel(float* __restrict__ h, T* __restrict__ rows, const T* __restrict__ table,
                                  const T* __restrict__ pair_table, const int* __restrict__ ids,
                                  const int* __restrict__ positions, const int* __restrict__ entry_of_token,
                                  const int* __restrict__ cu_q, const int* __restrict__ state_slot,
                                  const int* __restrict__ prev_token, float scale, int buckets, int mul_prev,
                                  int mul_cur, int D, int V, const int* __restrict__ pending, int n_pending,
                                  int* status) {
  ccb::pdl_begin();
  const int t = blockIdx.x;
  float* out = h + (size_t)t * D;
  T* out2 = rows ? rows + (size_t)t * D : nullptr;
  const int e = entry_of_token[t];
  int id = ids[t];
  if (id < 0 && pending != nullptr && -1 - id < n_pending) id = pending[-1 - id];
  if (e < 0 || id < 0 || id >= V) {
    if (e >= 0 && threadIdx.x == 0) set_status(status, CCB_ST_BAD_TOKEN);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      out[d] = 0.f;
      if (out2) out2[d] = from_f32<T>(0.f);
    }
    return;
  }
  const T* pr = nullptr;
  if (pair_table != nullptr) {
    int row = buckets;
    if (positions[t] > 0) {
      int prev;
      if (t > cu_q[e]) {
        prev = ids[t - 1];
      } else {
        const int slot = state_slot[e];
        prev = slot >= 0 ? prev_token[slot] : 0;
      }
      if (prev < 0 || prev >= V) {
        if (threadIdx.x == 0) set_status(status, CCB_ST_BAD_TOKEN);
        prev = 0;
      }
      row = (int)(((long long)prev * mul_prev + (long long)id * mul_cur) % buckets);
    }
    pr = pair_table + (size_t)row * D;
  }
  const T* er = table + (size_t)id * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = to_f32(er[d]) * scale;
    if (pr) v += to_f32(pr[d]);
    out[d] = v;
    if (out2) out2[d] = from_f32<T>(v);
  }
}

__global__ void embed_pair_commit_kernel(const int* __restrict__ ids, const int* __restrict__ cu_q,
                                         const int* __restrict__ state_slot, int* __restrict__ prev_token,
                                         int n_entries, int n_slots, const int* __restrict__ pending, int n_pending) {
  ccb::pdl_begin();
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_entries) return;
  const int slot = state_slot[e];
  const int n = cu_q[e + 1] - cu_q[e];
  if (slot < 0 || slot >= n_slots || n <= 0) return;
  int id = ids[cu_q[e + 1] - 1];
  if (id < 0 && pending != nullptr && -1 - id < n_pending) id = pending[-1 - id];
  prev_token[slot] = id;
}

CCB_API int ccb_embed_pair(float* h, void* rows, const void* table, const void* pair_table, const int* ids,
                           const int* positions, const int* entry_of_token, const int* cu_q, const int* state_slot,
                           int* prev_token, float scale, int buckets, int mul_prev, int mul_cur, int T_, int n_entries,
                           int n_slots, int D, int V, int dtype, const int* pending, int n_pending, int* status,
                           cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (D <= 0 || V <= 0 || (pair_table != nullptr && (buckets <= 0 || mul_prev < 0 || mul_cur < 0)))
    return CCB_REFUSE_SIZE;
  if (pair_table != nullptr && prev_token == nullptr) return CCB_REFUSE_ARG;
  const int threads = D >= 1024 ? 256 : 128;
  if (dtype == CCB_F32)
    ccb_launch(embed_pair_kernel<float>, T_, threads, 0, stream, h, (float*)rows, (const float*)table,
               (const float*)pair_table, ids, positions, entry_of_token, cu_q, state_slot, (const int*)prev_token, scale,
               buckets, mul_prev, mul_cur, D, V, pending, n_pending, status);
  else if (dtype == CCB_BF16)
    ccb_launch(embed_pair_kernel<__nv_bfloat16>, T_, threads, 0, stream, h, (__nv_bfloat16*)rows,
               (const __nv_bfloat16*)table, (const __nv_bfloat16*)pair_table, ids, positions, entry_of_token, cu_q,
               state_slot, (const int*)prev_token, scale, buckets, mul_prev, mul_cur, D, V, pending, n_pending, status);
  else
    return CCB_REFUSE_DTYPE;
  int rc = ccb_launch_status();
  if (rc != 0 || pair_table == nullptr || n_entries <= 0) return rc;
  ccb_launch(embed_pair_commit_kernel, (n_entries + 127) / 128, 128, 0, stream, ids, cu_q, state_slot, prev_token,
             n_entries, n_slots, pending, n_pending);
  return ccb_launch_status();
}

// ---------------------------------------------------------------------------------------------
// act = relu(x)^2, elementwise (the activation of a feed-forward without a gate).
template <typename T>
__global__ void relu_squared_kernel(T* __restrict__ act, const T* __restrict__ x, size_t total) {
  ccb::pdl_begin();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const float v = fmaxf(to_f32(x[i]), 0.f);
    act[i] = from_f32<T>(v * v);
  }
}

__global__ void relu_squared_bf16x8_kernel(uint4* __restrict__ act, const uint4* __restrict__ x, size_t total8) {
  ccb::pdl_begin();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 a = x[i];
    const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 f = __bfloat1622float2(ah[e]);
      f.x = fmaxf(f.x, 0.f);
      f.y = fmaxf(f.y, 0.f);
      oh[e] = __floats2bfloat162_rn(f.x * f.x, f.y * f.y);
    }
    act[i] = o;
  }
}

CCB_API int ccb_relu_squared(void* act, const void* x, long long total, int dtype, cudaStream_t stream) {
  if (total <= 0) return 0;
  const int threads = 256;
  if (dtype == CCB_BF16 && total % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(act) | reinterpret_cast<uintptr_t>(x)) & 15) == 0) {
    const size_t total8 = (size_t)total / 8;
    const size_t want = (total8 + threads - 1) / threads;
    ccb_launch(relu_squared_bf16x8_kernel, (int)(want < 148 * 32 ? want : 148 * 32), threads, 0, stream, (uint4*)act,
               (const uint4*)x, total8);
    return ccb_launch_status();
  }
  const size_t want = ((size_t)total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
  if (dtype == CCB_F32)
    ccb_launch(relu_squared_kernel<float>, blocks, threads, 0, stream, (float*)act, (const float*)x, (size_t)total);
  else if (dtype == CCB_BF16)
    ccb_launch(relu_squared_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16*)act,
               (const __nv_bfloat16*)x, (size_t)total);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// ---------------------------------------------------------------------------------------------
// out = sa * a + sb * b, elementwise in float (a pair of mixers on the same rows, each with a constant factor).
template <typename T>
__global__ void scaled_sum_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, float sa,
                                  float sb, size_t total) {
  ccb::pdl_begin();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(fmaf(sa, to_f32(a[i]), sb * to_f32(b[i])));
}

CCB_API int ccb_scaled_sum(void* out, const void* a, const void* b, float sa, float sb, long long total, int dtype,
                           cudaStream_t stream) {
  if (total <= 0) return 0;
  const int threads = 256;
  const size_t want = ((size_t)total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
  if (dtype == CCB_F32)
    ccb_launch(scaled_sum_kernel<float>, blocks, threads, 0, stream, (float*)out, (const float*)a, (const float*)b, sa,
               sb, (size_t)total);
  else if (dtype == CCB_BF16)
    ccb_launch(scaled_sum_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16*)out,
               (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, sa, sb, (size_t)total);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}
