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
// (src/infer/kv/paged_cache.py:40-43,90-91). slot_map == null with caches given writes token t's k and v to
// row t (dense [T, nkv, D] outputs, for a position encoding that is applied by a kernel of its own before
// the cache write); without caches nothing is written (a layer that reads another layer's cache). A negative
// slot is skipped too. cos_t == null: no rotation (bias and the split only). A position outside the tables
// is never read: the row is clamped (a memory guard) and `error`, when given, is set to 31, which the host
// turns into an exception; the engine refuses such a step before it launches.
#include "common.cuh"

namespace tmk {

// The table row of a position. Positions outside [0, n_pos) never index the tables: the row is clamped and
// the error word (when there is one) raised.
__device__ __forceinline__ int rope_position(int pos, int n_pos, int* error) {
  if (pos >= 0 && pos < n_pos) return pos;
  if (error && threadIdx.x == 0) atomicCAS(error, 0, 31);
  return pos < 0 ? 0 : n_pos - 1;
}

template <typename TIn, typename T>
__global__ void qkv_rope_write_kernel(const TIn* __restrict__ qkv, const float* __restrict__ bias,
                                      const int* __restrict__ positions, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, const int* __restrict__ slot_map,
                                      T* __restrict__ q_out, T* __restrict__ kcache, T* __restrict__ vcache,
                                      int nh, int nkv, int D, int n_pos, int* __restrict__ error) {
  pdl_launch_dependents();                     // (the kernel behind this one may start its own preparations)
  const int t = blockIdx.x;
  const int half = D >> 1;
  const int heads = nh + 2 * nkv;
  const int width = heads * D;
  const TIn* row = qkv + (size_t)t * width;
  const int pos = rope_position(cos_t ? positions[t] : 0, n_pos, error);
  const int slot = slot_map ? slot_map[t] : (kcache ? t : -1);
  for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx - h * half;
    const int c0 = h * D + i, c1 = c0 + half;
    float x1 = to_float(row[c0]), x2 = to_float(row[c1]);
    if (bias) {
      x1 += bias[c0];
      x2 += bias[c1];
    }
    float o1 = x1, o2 = x2;
    if (cos_t && h < nh + nkv) {
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

// The same, four rotation pairs per thread (head sizes that are multiples of 8, 16-byte aligned rows).
template <typename TIn, typename T>
__global__ void qkv_rope_write_vec_kernel(const TIn* __restrict__ qkv, const float* __restrict__ bias,
                                          const int* __restrict__ positions, const float* __restrict__ cos_t,
                                          const float* __restrict__ sin_t, const int* __restrict__ slot_map,
                                          T* __restrict__ q_out, T* __restrict__ kcache, T* __restrict__ vcache,
                                          int nh, int nkv, int D, int n_pos, int* __restrict__ error) {
  pdl_launch_dependents();                     // (the kernel behind this one may start its own preparations)
  pdl_wait();                                  // the product comes from the kernel in front of this one
  const int t = blockIdx.x;
  const int half = D >> 1, quads = half >> 2;
  const int heads = nh + 2 * nkv;
  const TIn* row = qkv + (size_t)t * heads * D;
  const int pos = rope_position(cos_t ? positions[t] : 0, n_pos, error);
  const int slot = slot_map ? slot_map[t] : (kcache ? t : -1);
  for (int idx = threadIdx.x; idx < heads * quads; idx += blockDim.x) {
    const int h = idx / quads, i = (idx - h * quads) * 4;
    const int c0 = h * D + i, c1 = c0 + half;
    float x1[4], x2[4], o1[4], o2[4];
    load4<TIn>(row + c0, x1);
    load4<TIn>(row + c1, x2);
    if (bias) {
      float b1[4], b2[4];
      load4<float>(bias + c0, b1);
      load4<float>(bias + c1, b2);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        x1[e] += b1[e];
        x2[e] += b2[e];
      }
    }
    if (cos_t && h < nh + nkv) {
      float cs[4], sn[4];
      load4<float>(cos_t + (size_t)pos * half + i, cs);
      load4<float>(sin_t + (size_t)pos * half + i, sn);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        o1[e] = __fadd_rn(__fmul_rn(x1[e], cs[e]), __fmul_rn(-x2[e], sn[e]));
        o2[e] = __fadd_rn(__fmul_rn(x2[e], cs[e]), __fmul_rn(x1[e], sn[e]));
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        o1[e] = x1[e];
        o2[e] = x2[e];
      }
    }
    T* dst = nullptr;
    if (h < nh) {
      dst = q_out + ((size_t)t * nh + h) * D;
    } else if (slot >= 0) {
      const bool is_k = h < nh + nkv;
      dst = (is_k ? kcache : vcache) + ((size_t)slot * nkv + (is_k ? h - nh : h - nh - nkv)) * D;
    }
    if (dst) {
      store4<T>(dst + i, o1);
      store4<T>(dst + i + half, o2);
    }
  }
}

// k, v [T, width] (width = kv_heads * head_dim) -> their cache slots (rows of `width` elements); a negative
// slot is skipped. For mixers whose position encoding ran as a kernel of its own on dense k.
template <typename T>
__global__ void kv_cache_write_kernel(const T* __restrict__ k, const T* __restrict__ v, const int* __restrict__ slot_map,
                                      T* __restrict__ kcache, T* __restrict__ vcache, int width) {
  const int t = blockIdx.x;
  const int slot = slot_map[t];
  if (slot < 0) return;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    kcache[(size_t)slot * width + i] = k[(size_t)t * width + i];
    vcache[(size_t)slot * width + i] = v[(size_t)t * width + i];
  }
}

}  // namespace tmk

extern "C" int tm_kv_cache_write(int dtype, const void* k, const void* v, const int* slot_map, void* kcache,
                                 void* vcache, int T, int width, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (width <= 0 || !slot_map || !kcache || !vcache) return TM_ERR_UNSUPPORTED_SHAPE;
  const int threads = width >= 256 ? 256 : (width + 31) / 32 * 32;
  if (dtype == TM_DTYPE_F32)
    tmk::kv_cache_write_kernel<float><<<T, threads, 0, stream>>>((const float*)k, (const float*)v, slot_map,
                                                                 (float*)kcache, (float*)vcache, width);
  else if (dtype == TM_DTYPE_BF16)
    tmk::kv_cache_write_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(
        (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, slot_map, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, width);
  else
    return TM_ERR_BAD_DTYPE;
  return tmk::launch_status();
}

// in_dtype: dtype of qkv (a 32-bit product may feed a bfloat16 cache); dtype: dtype of q_out and caches.
extern "C" int tm_qkv_rope_write(int in_dtype, int dtype, const void* qkv, const float* bias,
                                 const int* positions, const float* cos_t, const float* sin_t,
                                 const int* slot_map, void* q_out, void* kcache, void* vcache, int T, int nh,
                                 int nkv, int D, int n_pos, int* error, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D % 2 || (cos_t == nullptr) != (sin_t == nullptr)) return TM_ERR_UNSUPPORTED_SHAPE;
  using bf16 = __nv_bfloat16;
  const uintptr_t all = reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(bias) |
                        reinterpret_cast<uintptr_t>(cos_t) | reinterpret_cast<uintptr_t>(sin_t) |
                        reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(kcache) |
                        reinterpret_cast<uintptr_t>(vcache);
  const bool vec = D % 8 == 0 && (all & 15) == 0;
  const int work = (nh + 2 * nkv) * (D / 2) / (vec ? 4 : 1);
  const int threads = work >= 256 ? 256 : ((work + 31) / 32) * 32;
#define TM_ROPE_LAUNCH(TIN, TOUT)                                                                            \
  do {                                                                                                       \
    if (vec)                                                                                                 \
      return tmk::launch_pdl(tmk::qkv_rope_write_vec_kernel<TIN, TOUT>, dim3(T), dim3(threads), 0, stream,   \
                             (const TIN*)qkv, bias, positions, cos_t, sin_t, slot_map, (TOUT*)q_out, (TOUT*)kcache, \
                             (TOUT*)vcache, nh, nkv, D, n_pos, error);                                       \
    else                                                                                                     \
      tmk::qkv_rope_write_kernel<TIN, TOUT><<<T, threads, 0, stream>>>(                                      \
          (const TIN*)qkv, bias, positions, cos_t, sin_t, slot_map, (TOUT*)q_out, (TOUT*)kcache,             \
          (TOUT*)vcache, nh, nkv, D, n_pos, error);                                                               \
  } while (0)
  if (in_dtype == TM_DTYPE_F32 && dtype == TM_DTYPE_F32)
    TM_ROPE_LAUNCH(float, float);
  else if (in_dtype == TM_DTYPE_BF16 && dtype == TM_DTYPE_BF16)
    TM_ROPE_LAUNCH(bf16, bf16);
  else if (in_dtype == TM_DTYPE_F32 && dtype == TM_DTYPE_BF16)
    TM_ROPE_LAUNCH(float, bf16);
  else
    return TM_ERR_BAD_DTYPE;
#undef TM_ROPE_LAUNCH
  return tmk::launch_status();
}
