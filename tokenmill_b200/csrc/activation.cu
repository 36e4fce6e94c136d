// SwiGLU activation over the fused gate/up product: out[t, i] = silu(gu[t, i]) * gu[t, I + i],
// silu(g) = g * sigmoid(g) (src/infer/model/layers.py:162-164; gate rows come first in the fused
// matrix). Arithmetic in 32-bit, one rounding to the output dtype. When I is a multiple of 8 (4 for
// float32) and the pointers are 16-byte aligned, each thread moves 16 bytes per access.
#include "common.cuh"

namespace tmk {

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, long long total) {
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / I;
    const int i = (int)(idx - t * I);
    out[idx] = from_float<T>(silu_mul(to_float(gu[t * 2 * I + i]), to_float(gu[t * 2 * I + I + i])));
  }
}

// 16 bytes per access: VEC elements (8 bfloat16 or 4 float32). One block works on a piece of one row (the row
// is the block's x index), so that no thread divides a 64-bit index; with bfloat16 outputs the quotient is a
// reciprocal and a multiply (2 ulp in float32, far below the output's rounding): with the exact division and the
// flat index the kernel was bound by instruction issue, not by memory.
template <typename T, int VEC>
__global__ void __launch_bounds__(128) swiglu_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int I) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (i >= I) return;
  const uint4 g = *reinterpret_cast<const uint4*>(gu + t * 2 * I + i);
  const uint4 u = *reinterpret_cast<const uint4*>(gu + t * 2 * I + I + i);
  uint4 o;
  const T* gp = reinterpret_cast<const T*>(&g);
  const T* up = reinterpret_cast<const T*>(&u);
  T* op = reinterpret_cast<T*>(&o);
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    const float gf = to_float(gp[e]), uf = to_float(up[e]);
    if constexpr (sizeof(T) == 2) op[e] = from_float<T>(__fdividef(gf, 1.0f + expf(-gf)) * uf);
    else op[e] = from_float<T>(silu_mul(gf, uf));
  }
  *reinterpret_cast<uint4*>(out + t * I + i) = o;
}

// SwiGLU over a gate/up product that arrives as float32 partial sums [S, T, 2 I] (a product whose K range was
// cut): the slices are added in index order, gate and up are rounded to bfloat16 as a library product would have
// left them, and out [T, I] = silu(gate) * up in bfloat16. I a multiple of 4.
__global__ void __launch_bounds__(256) swiglu_partials_kernel(const float* __restrict__ parts, int S, long long stride,
                                                              __nv_bfloat16* __restrict__ out, int I, long long total) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int per_row = I / 4;
  const long long t = idx / per_row;
  const int i = (int)(idx - t * per_row) * 4;
  float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < S; ++s) {
    const float* row = parts + (size_t)s * stride + (size_t)t * 2 * I;
    const float4 a = *reinterpret_cast<const float4*>(row + i), b = *reinterpret_cast<const float4*>(row + I + i);
    g[0] += a.x; g[1] += a.y; g[2] += a.z; g[3] += a.w;
    u[0] += b.x; u[1] += b.y; u[2] += b.z; u[3] += b.w;
  }
  float o[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float gf = to_float(from_float<__nv_bfloat16>(g[e])), uf = to_float(from_float<__nv_bfloat16>(u[e]));
    o[e] = silu_mul(gf, uf);
  }
  store4<__nv_bfloat16>(out + t * I + i, o);
}

template <typename T>
int launch_swiglu(const void* gu, void* out, int T_, int I, cudaStream_t stream) {
  constexpr int VEC = 16 / sizeof(T);
  const int threads = 256;
  const bool aligned = ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (I % VEC == 0 && aligned) {
    const int per_row = I / VEC;
    return launch_pdl(swiglu_vec_kernel<T, VEC>, dim3(T_, (per_row + 127) / 128), dim3(128), 0, stream, (const T*)gu,
                      (T*)out, I);
  } else {
    const long long total = (long long)T_ * I;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    swiglu_kernel<T><<<(int)blocks, threads, 0, stream>>>((const T*)gu, (T*)out, I, total);
  }
  return launch_status();
}

}  // namespace tmk

extern "C" int tm_swiglu(int dtype, const void* gu, void* out, int T, int I, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dtype == TM_DTYPE_F32) return tmk::launch_swiglu<float>(gu, out, T, I, stream);
  if (dtype == TM_DTYPE_BF16) return tmk::launch_swiglu<__nv_bfloat16>(gu, out, T, I, stream);
  return TM_ERR_BAD_DTYPE;
}

// parts [S, T, 2 I] float32 (slice stride `stride` floats) -> out [T, I] bfloat16; I a multiple of 4.
extern "C" int tm_swiglu_partials(const float* parts, int S, long long stride, void* out, int T, int I,
                                  cudaStream_t stream) {
  if (T <= 0) return 0;
  if (S <= 0 || I % 4 || ((reinterpret_cast<uintptr_t>(parts) | reinterpret_cast<uintptr_t>(out)) & 15) || stride % 4)
    return TM_ERR_UNSUPPORTED_SHAPE;
  const long long total = (long long)T * (I / 4);
  return tmk::launch_pdl(tmk::swiglu_partials_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, parts, S,
                         stride, (__nv_bfloat16*)out, I, total);
}
