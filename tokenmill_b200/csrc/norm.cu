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
#include "common.cuh"

namespace tmk {

template <typename T>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(
    float* __restrict__ resid, const T* __restrict__ branch, const float* __restrict__ partials,
    int n_partials, long long partial_stride, const int* __restrict__ ids, const T* __restrict__ table,
    const int* __restrict__ rows, const float* __restrict__ weight, float eps, T* __restrict__ out, int H) {
  extern __shared__ float xs[];  // H floats + 32 for the reduction
  float* red = xs + H;
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float x;
    if (ids) {
      x = to_float(table[(size_t)ids[src] * H + i]);
    } else {
      x = resid[(size_t)src * H + i];
      if (branch) x += to_float(branch[(size_t)src * H + i]);
      if (partials) {
        float acc = 0.f;
        for (int p = 0; p < n_partials; ++p) acc += partials[(size_t)p * partial_stride + (size_t)src * H + i];
        x += acc;
      }
    }
    if (!rows && (ids || branch || partials)) resid[(size_t)src * H + i] = x;
    xs[i] = x;
    ss += x * x;
  }
  const float total = block_sum(ss, red);
  const float rstd = 1.0f / sqrtf(total / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const T normed = from_float<T>(xs[i] * rstd);
    out[(size_t)r * H + i] = from_float<T>(weight[i] * to_float(normed));
  }
}

template <typename T>
int launch_add_rmsnorm(float* resid, const void* branch, const float* partials, int n_partials,
                       long long partial_stride, const int* ids, const void* table, const int* rows,
                       const float* weight, float eps, void* out, int n_rows, int H, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t smem = (size_t)(H + 32) * sizeof(float);
  if (smem > 200 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  add_rmsnorm_kernel<T><<<n_rows, 256, smem, stream>>>(resid, (const T*)branch, partials, n_partials,
                                                       partial_stride, ids, (const T*)table, rows, weight, eps,
                                                       (T*)out, H);
  return launch_status();
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
