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
// tm_attention_combine merges the splits in index order. The order of all sums depends only on the
// request's own length.
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
    float* __restrict__ part_ml, int nh, int nkv, int page_size, float scale_log2, int window, int split_keys,
    int max_splits) {
  extern __shared__ __align__(128) unsigned char smem[];
  pdl_launch_dependents();
  pdl_wait();                                  // q and this step's keys and values come from the kernel before
  const int s = blockIdx.x;
  const int q_start = cu_q[s];
  decode_attention_unit<D>(q, kcache, vcache, block_table + (size_t)s * bt_stride, q_start, cu_q[s + 1] - q_start,
                           kv_before[s], blockIdx.y, blockIdx.z, part_acc, part_ml, nh, nkv, page_size, scale_log2,
                           window, split_keys, max_splits, smem, threadIdx.x, [] { __syncthreads(); });
}

template <int D>
int launch_decode_attention(const void* q, const void* kcache, const void* vcache, const int* block_table,
                            int bt_stride, const int* cu_q, const int* kv_before, int n_seqs, float* part_acc,
                            float* part_ml, int nh, int nkv, int page_size, float scale, int window, int split_keys,
                            int max_splits, cudaStream_t stream) {
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
                    kv_before, part_acc, part_ml, nh, nkv, page_size, scale * 1.4426950408889634f, window,
                    split_keys, max_splits);
}

}  // namespace tmk

// q [T, nh, D] bfloat16; caches [pages, page_size, nkv, D] bfloat16. Every request must bring at most
// 16 / (nh / nkv) tokens. Partials go to part_acc [T*nh, max_splits, D] and part_ml [T*nh, max_splits, 2];
// tm_attention_combine turns them into the output. Head sizes 64 and 128.
extern "C" int tm_decode_attention_bf16(const void* q, const void* kcache, const void* vcache,
                                        const int* block_table, int bt_stride, const int* cu_q,
                                        const int* kv_before, int n_seqs, float* part_acc, float* part_ml, int nh,
                                        int nkv, int D, int page_size, float scale, int window, int split_keys,
                                        int max_splits, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (nkv <= 0 || nh % nkv || nh / nkv > 16 || page_size <= 0) return TM_ERR_UNSUPPORTED_SHAPE;
  if (split_keys <= 0 || split_keys % tmk::kDecBN || max_splits <= 0) return TM_ERR_UNSUPPORTED_SHAPE;
  if (!part_acc || !part_ml) return TM_ERR_SCRATCH_TOO_SMALL;
  if (D == 64)
    return tmk::launch_decode_attention<64>(q, kcache, vcache, block_table, bt_stride, cu_q, kv_before, n_seqs,
                                            part_acc, part_ml, nh, nkv, page_size, scale, window, split_keys,
                                            max_splits, stream);
  if (D == 128)
    return tmk::launch_decode_attention<128>(q, kcache, vcache, block_table, bt_stride, cu_q, kv_before, n_seqs,
                                             part_acc, part_ml, nh, nkv, page_size, scale, window, split_keys,
                                             max_splits, stream);
  return TM_ERR_UNSUPPORTED_SHAPE;
}
