// Fused embedding-gather / residual-add + RMSNorm.
//
// The residual stream is kept in 32-bit. One block handles one row:
//   x = table[ids[row]]                 (embedding mode: the stream starts here), or
//   x = resid[row] + branch[row]        (add mode; the sum is taken and stored in 32-bit), or
//   x = resid[row]                      (norm only)
//   y = weight * cast(x * rsqrt(mean(x^2) + eps))
// The formula is the reference's RMSNorm (src/infer/model/layers.py:35-44): statistics in 32-bit,
// the normalised value cast to the activation dtype BEFORE the weight multiply; the residual adds are
// src/infer/model/qwen2.py:22-23 and the embedding gather qwen2.py:46. With `rows` given, only those
// rows are normed and written densely (the final norm before the output matrix, engine/model_runner.py:96)
// and the residual stream is left untouched. `branch` may also be a stack of `n_partials` 32-bit partial
// products [n_partials, n_tokens, H] from a split-K matrix product; they are summed in index order.
// Rows whose width is a multiple of 4 move four elements per access; the order of the row's sum of
// squares is fixed by the width and the block size alone.
#include <type_traits>

#include "common.cuh"

namespace tmk {

template <typename T, int VEC>   // VEC = 1 or 4 elements per access
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(
    float* __restrict__ resid, const T* __restrict__ branch, const float* __restrict__ partials,
    int n_partials, long long partial_stride, const int* __restrict__ ids, const T* __restrict__ table,
    const int* __restrict__ rows, const float* __restrict__ weight, float eps, T* __restrict__ out, int H) {
  extern __shared__ __align__(16) float xs[];  // H floats + 32 for the reduction
  float* red = xs + H;
  pdl_launch_dependents();
  pdl_wait();                                  // everything this kernel reads comes from the kernels before it
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const bool write_back = !rows && (ids || branch || partials);
  float ss = 0.f;
  for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
    float x[VEC];
    if (ids) {
      const T* p = table + (size_t)ids[src] * H + i;
      if constexpr (VEC == 4) load4<T>(p, x); else x[0] = to_float(p[0]);
    } else {
      const float* p = resid + (size_t)src * H + i;
      if constexpr (VEC == 4) load4<float>(p, x); else x[0] = p[0];
      if (branch) {
        float b[VEC];
        const T* q = branch + (size_t)src * H + i;
        if constexpr (VEC == 4) load4<T>(q, b); else b[0] = to_float(q[0]);
#pragma unroll
        for (int e = 0; e < VEC; ++e) x[e] += b[e];
      }
      if (partials) {
        float acc[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
        for (int p2 = 0; p2 < n_partials; ++p2) {
          float v[VEC];
          const float* q = partials + (size_t)p2 * partial_stride + (size_t)src * H + i;
          if constexpr (VEC == 4) load4<float>(q, v); else v[0] = q[0];
#pragma unroll
          for (int e = 0; e < VEC; ++e) acc[e] += v[e];
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) x[e] += acc[e];
      }
    }
    if (write_back) {
      float* p = resid + (size_t)src * H + i;
      if constexpr (VEC == 4) store4<float>(p, x); else p[0] = x[0];
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      xs[i + e] = x[e];
      ss += x[e] * x[e];
    }
  }
  const float total = block_sum(ss, red);
  const float rstd = 1.0f / sqrtf(total / (float)H + eps);
  for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
    float y[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) y[e] = weight[i + e] * to_float(from_float<T>(xs[i + e] * rstd));
    T* p = out + (size_t)r * H + i;
    if constexpr (VEC == 4) store4<T>(p, y); else p[0] = from_float<T>(y[0]);
  }
}

// The same, one WARP per row: the row lives in the warp's registers (CH chunks of 4 elements per lane), so
// there is no shared memory and no block-level synchronisation, and a few thousand rows are in flight on the
// chip at once. One block per row left a long prompt's norm bound by the latency of its load, reduce and store
// chain, two waves deep. Rows up to 128 CH wide whose width is a multiple of 4; the order of the sum of
// squares (lane-wise over the chunks, then the butterfly across lanes) is fixed by the width alone.
template <typename T, int CH>
__global__ void __launch_bounds__(128) add_rmsnorm_warp_kernel(
    float* __restrict__ resid, const T* __restrict__ branch, const float* __restrict__ partials,
    int n_partials, long long partial_stride, const int* __restrict__ ids, const T* __restrict__ table,
    const int* __restrict__ rows, const float* __restrict__ weight, float eps, T* __restrict__ out, int H,
    int n_rows) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  float w[CH][4];
#pragma unroll
  for (int c = 0; c < CH; ++c) {               // the weights depend on no earlier kernel
    const int i = (c * 32 + lane) * 4;
    if (i < H) load4<float>(weight + i, w[c]);
  }
  pdl_launch_dependents();
  pdl_wait();
  if (r >= n_rows) return;
  const int src = rows ? rows[r] : r;
  const bool write_back = !rows && (ids || branch || partials);
  float x[CH][4];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = (c * 32 + lane) * 4;
    if (i >= H) continue;
    if (ids) {
      load4<T>(table + (size_t)ids[src] * H + i, x[c]);
    } else {
      load4<float>(resid + (size_t)src * H + i, x[c]);
      if (branch) {
        float b[4];
        load4<T>(branch + (size_t)src * H + i, b);
#pragma unroll
        for (int e = 0; e < 4; ++e) x[c][e] += b[e];
      }
      if (partials) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int p2 = 0; p2 < n_partials; ++p2) {
          float v[4];
          load4<float>(partials + (size_t)p2 * partial_stride + (size_t)src * H + i, v);
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[e] += v[e];
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) x[c][e] += acc[e];
      }
    }
    if (write_back) store4<float>(resid + (size_t)src * H + i, x[c]);
#pragma unroll
    for (int e = 0; e < 4; ++e) ss += x[c][e] * x[c][e];
  }
  const float total = warp_sum(ss);
  const float rstd = 1.0f / sqrtf(total / (float)H + eps);
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = (c * 32 + lane) * 4;
    if (i >= H) continue;
    float y[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) y[e] = w[c][e] * to_float(from_float<T>(x[c][e] * rstd));
    store4<T>(out + (size_t)r * H + i, y);
  }
}

template <typename T, int CH, typename... Args>
int launch_add_rmsnorm_warp(int n_rows, cudaStream_t stream, Args... args) {
  const int warps = 4;
  return launch_pdl(add_rmsnorm_warp_kernel<T, CH>, dim3((n_rows + warps - 1) / warps), dim3(32 * warps), 0, stream,
                    args..., n_rows);
}

template <typename T>
int launch_add_rmsnorm(float* resid, const void* branch, const float* partials, int n_partials,
                       long long partial_stride, const int* ids, const void* table, const int* rows,
                       const float* weight, float eps, void* out, int n_rows, int H, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t smem = (size_t)(H + 32) * sizeof(float);
  if (smem > 200 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
  const uintptr_t all = reinterpret_cast<uintptr_t>(resid) | reinterpret_cast<uintptr_t>(branch) |
                        reinterpret_cast<uintptr_t>(partials) | reinterpret_cast<uintptr_t>(table) |
                        reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(weight);
  const bool vec = H % 4 == 0 && (all & 15) == 0 && (partial_stride % 4 == 0);
  // A warp per row pays for long prompts of narrow rows (2,048 rows of 896: 5.2 us against 6.1; 4,096: 8.5 against
  // 10.3); a block per row wins everywhere else (64 rows of 896: 2.2 us against 4.6; rows of 1,536: 2.8 against 7.1,
  // and 7.9 against 12.4 at 2,048 rows, where a lane holds too much of the row). The two sum the squares in different
  // orders, so the 32-bit path, whose results do not move with the cut of a step, stays with one of them.
  if (vec && std::is_same<T, __nv_bfloat16>::value && H <= 128 * 8 && n_rows >= 1536) {
    const int chunks = (H + 127) / 128;
#define TM_NORM_WARP(CH)                                                                                          \
  return launch_add_rmsnorm_warp<T, CH>(n_rows, stream, resid, (const T*)branch, partials, n_partials, partial_stride, \
                                        ids, (const T*)table, rows, weight, eps, (T*)out, H)
    if (chunks <= 1) TM_NORM_WARP(1);
    if (chunks <= 2) TM_NORM_WARP(2);
    if (chunks <= 4) TM_NORM_WARP(4);
    TM_NORM_WARP(8);
#undef TM_NORM_WARP
  }
  auto kern = vec ? add_rmsnorm_kernel<T, 4> : add_rmsnorm_kernel<T, 1>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  // (256 threads a row: larger blocks gain half a microsecond at 8 rows of 3,584 and lose a factor at 2,048 rows.)
  return launch_pdl(kern, dim3(n_rows), dim3(256), smem, stream, resid, (const T*)branch, partials, n_partials,
                    partial_stride, ids, (const T*)table, rows, weight, eps, (T*)out, H);
}

}  // namespace tmk

// resid: [n_tokens, H] float (read, and written unless `rows`); branch: [n_tokens, H] dtype or null;
// partials: [n_partials, n_tokens, H] float or null; ids/table: embedding mode when ids != null;
// rows: [n_rows] int or null; weight: [H] float; out: [n_rows, H] dtype.
extern "C" int tm_add_rmsnorm(int dtype, float* resid, const void* branch, const float* partials,
                              int n_partials, long long partial_stride, const int* ids, const void* table,
                              const int* rows, const float* weight, float eps, void* out, int n_rows, int H,
                              cudaStream_t stream) {
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_add_rmsnorm<float>(resid, branch, partials, n_partials, partial_stride, ids, table, rows,
                                          weight, eps, out, n_rows, H, stream);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_add_rmsnorm<__nv_bfloat16>(resid, branch, partials, n_partials, partial_stride, ids, table,
                                                  rows, weight, eps, out, n_rows, H, stream);
  return TM_ERR_BAD_DTYPE;
}
