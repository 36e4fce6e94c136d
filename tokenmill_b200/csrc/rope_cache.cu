// Bias + rotate-half position encoding + paged key/value write, in one pass over the QKV product.
//
// Input  qkv [T, (nh + 2*nkv) * D]: rows of [q heads | k heads | v heads] as the fused projection
//        lays them out (src/infer/model/layers.py:143-147).
// For q and k (src/infer/model/layers.py:55-64, rotate_half(x) = cat[-x[D/2:], x[:D/2]]):
//        out[i]       = x[i]       * cos[pos][i] - x[i + D/2] * sin[pos][i]
//        out[i + D/2] = x[i + D/2] * cos[pos][i] + x[i]       * sin[pos][i]
// with 32-bit cos/sin tables [P, D/2] (the reference's tables repeat each half, layers.py:47-52).
// The products and the sum are rounded separately (no fused multiply-add), as the reference's
// elementwise expression rounds them. q goes to q_out [T, nh, D]; k and v go straight to their slot
// of the paged cache, slot = page * page_size + offset, rows of [nkv, D]
// (src/infer/kv/paged_cache.py:40-43,90-91). slot_map == null skips the cache write (a layer that
// reads another layer's cache). A negative slot is skipped too.
#include "common.cuh"

namespace tmk {

template <typename TIn, typename T>
__global__ void qkv_rope_write_kernel(const TIn* __restrict__ qkv, const float* __restrict__ bias,
                                      const int* __restrict__ positions, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, const int* __restrict__ slot_map,
                                      T* __restrict__ q_out, T* __restrict__ kcache, T* __restrict__ vcache,
                                      int nh, int nkv, int D, int n_pos) {
  const int t = blockIdx.x;
  const int half = D >> 1;
  const int heads = nh + 2 * nkv;
  const int width = heads * D;
  const TIn* row = qkv + (size_t)t * width;
  int pos = positions[t];
  if (pos < 0) pos = 0;
  if (pos >= n_pos) pos = n_pos - 1;
  const int slot = slot_map ? slot_map[t] : -1;
  for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx - h * half;
    const int c0 = h * D + i, c1 = c0 + half;
    float x1 = to_float(row[c0]), x2 = to_float(row[c1]);
    if (bias) {
      x1 += bias[c0];
      x2 += bias[c1];
    }
    float o1 = x1, o2 = x2;
    if (h < nh + nkv) {
      const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
      o1 = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(-x2, s));
      o2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
    }
    if (h < nh) {
      T* dst = q_out + ((size_t)t * nh + h) * D;
      dst[i] = from_float<T>(o1);
      dst[i + half] = from_float<T>(o2);
    } else if (slot >= 0) {
      const bool is_k = h < nh + nkv;
      const int kh = is_k ? h - nh : h - nh - nkv;
      T* dst = (is_k ? kcache : vcache) + ((size_t)slot * nkv + kh) * D;
      dst[i] = from_float<T>(o1);
      dst[i + half] = from_float<T>(o2);
    }
  }
}

}  // namespace tmk

// in_dtype: dtype of qkv (a 32-bit product may feed a bfloat16 cache); dtype: dtype of q_out and caches.
extern "C" int tm_qkv_rope_write(int in_dtype, int dtype, const void* qkv, const float* bias,
                                 const int* positions, const float* cos_t, const float* sin_t,
                                 const int* slot_map, void* q_out, void* kcache, void* vcache, int T, int nh,
                                 int nkv, int D, int n_pos, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D % 2) return TM_ERR_UNSUPPORTED_SHAPE;
  const int work = (nh + 2 * nkv) * (D / 2);
  const int threads = work >= 256 ? 256 : ((work + 31) / 32) * 32;
  using bf16 = __nv_bfloat16;
  if (in_dtype == TM_DTYPE_F32 && dtype == TM_DTYPE_F32)
    tmk::qkv_rope_write_kernel<float, float><<<T, threads, 0, stream>>>(
        (const float*)qkv, bias, positions, cos_t, sin_t, slot_map, (float*)q_out, (float*)kcache,
        (float*)vcache, nh, nkv, D, n_pos);
  else if (in_dtype == TM_DTYPE_BF16 && dtype == TM_DTYPE_BF16)
    tmk::qkv_rope_write_kernel<bf16, bf16><<<T, threads, 0, stream>>>(
        (const bf16*)qkv, bias, positions, cos_t, sin_t, slot_map, (bf16*)q_out, (bf16*)kcache, (bf16*)vcache,
        nh, nkv, D, n_pos);
  else if (in_dtype == TM_DTYPE_F32 && dtype == TM_DTYPE_BF16)
    tmk::qkv_rope_write_kernel<float, bf16><<<T, threads, 0, stream>>>(
        (const float*)qkv, bias, positions, cos_t, sin_t, slot_map, (bf16*)q_out, (bf16*)kcache, (bf16*)vcache,
        nh, nkv, D, n_pos);
  else
    return TM_ERR_BAD_DTYPE;
  return tmk::launch_status();
}
