// Decode attention over the paged cache on tensor cores (bfloat16 in, float32 softmax and accumulate).
//
// For steps whose requests each bring so few query rows that one request and one kv head fit a
// single 16-row tile: rows are (token, head-in-group) pairs, q_len * G <= 16 (a decoded token with
// up to 16 query heads per kv head, or a two-token portion with 7). Semantics are those of
// attention_paged.cu (src/infer/model/layers.py:100-124, src/infer/kv/context.py:77-79): keys
// j <= p of the same request, j > p - window if a window is set, softmax in 32-bit.
//
// One block of 4 warps per (request, kv head, key split). Keys are cut at absolute multiples of
// split_keys (a multiple of 64); within a split, blocks of 64 keys stream through shared memory with
// cp.async (two stages), and the 4 warps take 16 keys each of every block, so the keys of one request
// are spread over 4 * splits warps. Each warp keeps an online-softmax state for its keys; the 4 states
// are merged in warp order through shared memory and written as one partial (max, sum, acc) per split;
// the block that finishes a (request, kv head) last merges the splits in index order and writes the head
// outputs (one arrival counter per pair, left at zero for the next launch), so no second kernel is needed.
// The order of all sums depends only on the request's own length.
//
// K tiles are read with ldmatrix (rows = keys), V tiles with ldmatrix.trans; rows of a tile are
// XOR-swizzled in 16-byte chunks so both reads are bank-conflict free. Matrix products are
// mma.sync.m16n8k16 (bf16 x bf16 -> f32): at 16 query rows per request the tile is far too small for
// a tcgen05 instruction (M >= 64), and the kernel is bound by memory latency, not by math.
#include "attention_decode_core.cuh"

namespace tmk {

template <int D>
__global__ void __launch_bounds__(kDecWarps * 32) decode_attention_bf16_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kcache,
    const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_table, int bt_stride,
    const int* __restrict__ cu_q, const int* __restrict__ kv_before, float* __restrict__ part_acc,
    float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out, int* __restrict__ done, int nh, int nkv,
    int page_size, float scale_log2, int window, int split_keys, int max_splits, int* __restrict__ error) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_last;
  pdl_launch_dependents();
  // (The request's lengths and block table are the step's inputs, copied before its first kernel: they and the
  // older keys and values may be read before the kernel in front of this one has finished.)
  const int s = blockIdx.x, kvh = blockIdx.y;
  const int q_start = cu_q[s], q_len = cu_q[s + 1] - q_start, before = kv_before[s];
  // What the host cannot check (the lengths live on the device): a request with more rows than a tile holds,
  // or with keys beyond the last split of the launch grid. Such a request's output would be incomplete; the
  // error word says so (32), the splits that exist are still merged and the counters still end at zero.
  if (threadIdx.x == 0 && blockIdx.z == 0 && kvh == 0 && error &&
      (q_len * (nh / nkv) > 16 || (q_len > 0 && (before + q_len - 1) / split_keys >= max_splits)))
    atomicCAS(error, 0, 32);
  const bool worked = decode_attention_unit<D>(q, kcache, vcache, block_table + (size_t)s * bt_stride, q_start, q_len,
                                               before, kvh, blockIdx.z, part_acc, part_ml, nh, nkv, page_size,
                                               scale_log2, window, split_keys, max_splits, smem, threadIdx.x,
                                               [] { __syncthreads(); }, [] { pdl_wait(); });
  if (!worked) {                               // no key of this request in this split (uniform over the block)
    pdl_wait();                                // (every kernel of the chain waits before it exits)
    return;
  }
  // How many splits hold keys for this (request, kv head): the last of them to finish merges all.
  const int G = nh / nkv;
  const int n_rows = min(q_len * G, 16);
  const int p_max = before + (n_rows - 1) / G;
  const int lo_all = window > 0 ? max(0, before - window + 1) : 0;
  const int z_last = min(p_max / split_keys, max_splits - 1);        // splits beyond the grid do not exist
  const int expected = z_last - lo_all / split_keys + 1;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&done[s * nkv + kvh], 1) == expected - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < n_rows * (D / 4); idx += kDecWarps * 32) {
    const int r = idx / (D / 4), d = (idx - r * (D / 4)) * 4;
    const size_t orow = (size_t)(q_start + r / G) * nh + kvh * G + r % G;
    const int p = before + r / G;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int z0 = lo / split_keys, z1 = min(p / split_keys, max_splits - 1);
    // One pass in split order: the running maximum rescales what has been summed so far. The loads do not
    // depend on the running state, so several splits are in flight at a time.
    float mx = -INFINITY, lsum = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int zz = z0; zz <= z1; ++zz) {
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + (orow * max_splits + zz) * 2));
      const float4 pa = __ldcg(reinterpret_cast<const float4*>(part_acc + (orow * max_splits + zz) * D + d));
      const float m_new = fmaxf(mx, ml.x);
      const float keep = mx == -INFINITY ? 0.f : expf(mx - m_new);
      const float w = ml.x == -INFINITY ? 0.f : expf(ml.x - m_new);
      lsum = lsum * keep + ml.y * w;
      acc[0] = acc[0] * keep + pa.x * w;
      acc[1] = acc[1] * keep + pa.y * w;
      acc[2] = acc[2] * keep + pa.z * w;
      acc[3] = acc[3] * keep + pa.w * w;
      mx = m_new;
    }
    const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
    uint2 o;
    o.x = pack_bf16(acc[0] * inv, acc[1] * inv);
    o.y = pack_bf16(acc[2] * inv, acc[3] * inv);
    *reinterpret_cast<uint2*>(out + orow * D + d) = o;
  }
  if (threadIdx.x == 0) done[s * nkv + kvh] = 0;
}

template <int D>
int launch_decode_attention(const void* q, const void* kcache, const void* vcache, const int* block_table,
                            int bt_stride, const int* cu_q, const int* kv_before, int n_seqs, float* part_acc,
                            float* part_ml, void* out, int* done, int nh, int nkv, int page_size, float scale,
                            int window, int split_keys, int max_splits, int* error, cudaStream_t stream) {
  const int kv_bytes = 2 * 2 * kDecBN * D * 2;
  const int merge_bytes = kDecWarps * 16 * (D + 2) * 4;
  const int smem = kv_bytes > merge_bytes ? kv_bytes : merge_bytes;
  auto kern = decode_attention_bf16_kernel<D>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
  }
  const dim3 grid(n_seqs, nkv, max_splits);
  return launch_pdl(kern, grid, dim3(kDecWarps * 32), (size_t)smem, stream, (const __nv_bfloat16*)q,
                    (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_table, bt_stride, cu_q,
                    kv_before, part_acc, part_ml, (__nv_bfloat16*)out, done, nh, nkv, page_size,
                    scale * 1.4426950408889634f, window, split_keys, max_splits, error);
}

}  // namespace tmk

// q, out [T, nh, D] bfloat16; caches [pages, page_size, nkv, D] bfloat16. Every request must bring at most
// 16 / (nh / nkv) tokens. Scratch: part_acc [T*nh, max_splits, D], part_ml [T*nh, max_splits, 2] float32, and
// done [n_seqs * nkv] ints that are zero before the first launch (the kernel leaves them zero). Head sizes 64
// and 128. max_splits * split_keys must exceed the longest context of the step; where it does not, or a request
// brings more rows than a tile, `error` (a device int that is zero; may be null) is set to 32 and that request's
// output is incomplete.
extern "C" int tm_decode_attention_bf16(const void* q, const void* kcache, const void* vcache,
                                        const int* block_table, int bt_stride, const int* cu_q,
                                        const int* kv_before, int n_seqs, float* part_acc, float* part_ml,
                                        void* out, int* done, int nh, int nkv, int D, int page_size, float scale,
                                        int window, int split_keys, int max_splits, int* error,
                                        cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (nkv <= 0 || nh % nkv || nh / nkv > 16 || page_size <= 0) return TM_ERR_UNSUPPORTED_SHAPE;
  if (split_keys <= 0 || split_keys % tmk::kDecBN || max_splits <= 0) return TM_ERR_UNSUPPORTED_SHAPE;
  if (!part_acc || !part_ml || !done || !out) return TM_ERR_SCRATCH_TOO_SMALL;
  if (D == 64)
    return tmk::launch_decode_attention<64>(q, kcache, vcache, block_table, bt_stride, cu_q, kv_before, n_seqs,
                                            part_acc, part_ml, out, done, nh, nkv, page_size, scale, window,
                                            split_keys, max_splits, error, stream);
  if (D == 128)
    return tmk::launch_decode_attention<128>(q, kcache, vcache, block_table, bt_stride, cu_q, kv_before, n_seqs,
                                             part_acc, part_ml, out, done, nh, nkv, page_size, scale, window,
                                             split_keys, max_splits, error, stream);
  return TM_ERR_UNSUPPORTED_SHAPE;
}
