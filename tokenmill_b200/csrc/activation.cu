// SwiGLU activation over the fused gate/up product: out[t, i] = silu(gu[t, i]) * gu[t, I + i],
// silu(g) = g * sigmoid(g) (src/infer/model/layers.py:162-164; gate rows come first in the fused
// matrix). Arithmetic in 32-bit, one rounding to the output dtype.
#include "common.cuh"

namespace tmk {

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, long long total) {
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_float(gu[t * 2 * I + i]);
    const float u = to_float(gu[t * 2 * I + I + i]);
    const float act = g / (1.0f + expf(-g));
    out[idx] = from_float<T>(act * u);
  }
}

}  // namespace tmk

extern "C" int tm_swiglu(int dtype, const void* gu, void* out, int T, int I, cudaStream_t stream) {
  if (T <= 0) return 0;
  const long long total = (long long)T * I;
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == TM_DTYPE_F32)
    tmk::swiglu_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gu, (float*)out, I, total);
  else if (dtype == TM_DTYPE_BF16)
    tmk::swiglu_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>((const __nv_bfloat16*)gu,
                                                                         (__nv_bfloat16*)out, I, total);
  else
    return TM_ERR_BAD_DTYPE;
  return tmk::launch_status();
}
