// Causal attention of prompt portions over the paged cache on tensor cores (bfloat16 in, float32
// softmax and accumulate), one pass, no partial results.
//
// Semantics as attention_paged.cu (src/infer/model/layers.py:72-107, src/infer/kv/context.py:63-76):
// the step's keys and values already sit in the cache; the query at absolute position p of a request
// reads that request's keys j <= p (and j > p - window if a window is set); query head h reads kv
// head h / G. Any mix of requests works (a decoded token is a portion of one), but the kernel is laid
// out for long portions: a block is one request's tile of 64 consecutive tokens and one query head,
// 4 warps of 16 rows. Keys stream through shared memory in blocks of 64 anchored at absolute positions
// 0, 64, 128, ... (cp.async, two stages); each warp multiplies its 16 queries with the whole block
// (ldmatrix + mma.sync.m16n8k16), keeps the online-softmax state in registers and adds P.V with V read
// through ldmatrix.trans. Because the key blocks are anchored at absolute positions, a row's sums
// run in the same order however the prompt was cut into portions.
//
// This is the mma.sync ("legacy tensor core") formulation; it reaches a fraction of what a tcgen05
// kernel with the accumulators in tensor memory would, and is the stand-in until that kernel exists.
#include "mma_util.cuh"

namespace tmk {

constexpr int kPfBM = 64;        // query tokens per block
constexpr int kPfBN = 64;        // keys per stage
constexpr int kPfWarps = 4;

template <int D>
__global__ void __launch_bounds__(kPfWarps * 32) prefill_attention_bf16_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kcache,
    const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_table, int bt_stride,
    const int* __restrict__ cu_q, const int* __restrict__ kv_before, const int* __restrict__ tile_seq,
    const int* __restrict__ tile_tok0, __nv_bfloat16* __restrict__ out, int nh, int nkv, int page_size,
    float scale_log2, int window) {
  constexpr int CH = D / 8;
  constexpr int KS = D / 16;
  constexpr int NT = D / 8;
  constexpr int TILE_BYTES = kPfBN * D * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t smem_base = smem_u32(smem);

  const int s = tile_seq[blockIdx.x];
  const int tok0 = tile_tok0[blockIdx.x];           // first token of the tile within the request's portion
  const int head = blockIdx.y;
  const int kvh = head / (nh / nkv);
  const int q_start = cu_q[s];
  const int q_len = cu_q[s + 1] - q_start;
  const int before = kv_before[s];
  if (tok0 >= q_len) return;
  const int n_tok = min(kPfBM, q_len - tok0);
  const int p_min = before + tok0, p_max = before + tok0 + n_tok - 1;
  const int j_lo = window > 0 ? max(0, p_min - window + 1) : 0;
  const int j_hi = p_max;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* table = block_table + (size_t)s * bt_stride;
  const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;      // rows (tokens of the tile) of this thread
  const int cpair = (lane & 3) * 2;

  uint32_t qa[KS][4];
  {
    const __nv_bfloat16* qr0 = r0 < n_tok ? q + ((size_t)(q_start + tok0 + r0) * nh + head) * D : nullptr;
    const __nv_bfloat16* qr1 = r1 < n_tok ? q + ((size_t)(q_start + tok0 + r1) * nh + head) * D : nullptr;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int c = ks * 16 + cpair;
      qa[ks][0] = qr0 ? *reinterpret_cast<const uint32_t*>(qr0 + c) : 0u;
      qa[ks][1] = qr1 ? *reinterpret_cast<const uint32_t*>(qr1 + c) : 0u;
      qa[ks][2] = qr0 ? *reinterpret_cast<const uint32_t*>(qr0 + c + 8) : 0u;
      qa[ks][3] = qr1 ? *reinterpret_cast<const uint32_t*>(qr1 + c + 8) : 0u;
    }
  }
  const int p_r0 = r0 < n_tok ? p_min + r0 : -1, p_r1 = r1 < n_tok ? p_min + r1 : -1;
  const int lo_r0 = window > 0 ? max(0, p_r0 - window + 1) : 0, lo_r1 = window > 0 ? max(0, p_r1 - window + 1) : 0;
  // Keys this warp's 16 rows can see at all (its rows are consecutive positions).
  const int warp_p_hi = min(p_max, p_min + warp * 16 + 15);
  const int warp_lo = window > 0 ? max(0, p_min + warp * 16 - window + 1) : 0;

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;

  const int kb_first = (j_lo / kPfBN) * kPfBN;
  const int n_blocks = (j_hi - kb_first) / kPfBN + 1;

  auto load_block = [&](int stage, int kb) {
    const uint32_t k_dst = smem_base + stage * 2 * TILE_BYTES, v_dst = k_dst + TILE_BYTES;
    for (int idx = tid; idx < kPfBN * CH; idx += kPfWarps * 32) {
      const int row = idx / CH, c = idx - row * CH;
      const int j = kb + row;
      const bool ok = j >= j_lo && j <= j_hi;
      size_t src = 0;
      if (ok) {
        const int page = table[j / page_size];
        src = (((size_t)page * page_size + (j % page_size)) * nkv + kvh) * D + c * 8;
      }
      const uint32_t off = row * (D * 2) + ((c ^ (row & 7)) << 4);
      cp_async16(k_dst + off, kcache + src, ok);
      cp_async16(v_dst + off, vcache + src, ok);
    }
  };

  load_block(0, kb_first);
  cp_async_commit();
  for (int b = 0; b < n_blocks; ++b) {
    const int kb = kb_first + b * kPfBN;
    const int stage = b & 1;
    if (b + 1 < n_blocks) {
      load_block(stage ^ 1, kb + kPfBN);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    // else: the warp has no rows, or nothing in this block is visible to them
    if (warp * 16 < n_tok && kb <= warp_p_hi && kb + kPfBN - 1 >= warp_lo) {
      const uint32_t k_base = smem_base + stage * 2 * TILE_BYTES, v_base = k_base + TILE_BYTES;
      float sc[8][4];
#pragma unroll
      for (int t = 0; t < 8; ++t) sc[t][0] = sc[t][1] = sc[t][2] = sc[t][3] = 0.f;
      {
        const int krow = (lane & 7) + ((lane >> 4) << 3);
        const int csel = (lane >> 3) & 1;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {                    // 16 keys at a time
            const int key = kk * 16 + krow;
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(k_base + key * (D * 2) + (((2 * ks + csel) ^ (key & 7)) << 4), b0, b1, b2, b3);
            mma_bf16_16816(sc[2 * kk], qa[ks], b0, b1);
            mma_bf16_16816(sc[2 * kk + 1], qa[ks], b2, b3);
          }
        }
      }
      // No mask is needed when every key of the block is visible to every row of the warp: the block
      // ends at or before the warp's first position and starts at or after its last row's window.
      const bool need_mask = kb + kPfBN - 1 > p_min + warp * 16 ||
                             (window > 0 && kb < max(0, p_min + warp * 16 + 15 - window + 1));
      float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
      for (int t = 0; t < 8; ++t)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = kb + t * 8 + cpair + e;
          bool ok0 = true, ok1 = true;
          if (need_mask) {
            ok0 = j <= p_r0 && j >= lo_r0;
            ok1 = j <= p_r1 && j >= lo_r1;
          }
          sc[t][e] = ok0 ? sc[t][e] * scale_log2 : -INFINITY;
          sc[t][2 + e] = ok1 ? sc[t][2 + e] * scale_log2 : -INFINITY;
          tmax0 = fmaxf(tmax0, sc[t][e]);
          tmax1 = fmaxf(tmax1, sc[t][2 + e]);
        }
      tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
      tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
      tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
      tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
      const float mn0 = fmaxf(m0, tmax0), mn1 = fmaxf(m1, tmax1);
      const float corr0 = mn0 == -INFINITY ? 1.f : exp2f(m0 - mn0), corr1 = mn1 == -INFINITY ? 1.f : exp2f(m1 - mn1);
      const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
      float ps0 = 0.f, ps1 = 0.f;
      uint32_t pa[4][4];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        float p[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            p[h][e] = exp2f(sc[2 * kk + h][e] - base0);            // masked entries are -inf: exp2 gives 0
            p[h][2 + e] = exp2f(sc[2 * kk + h][2 + e] - base1);
            ps0 += p[h][e];
            ps1 += p[h][2 + e];
          }
        pa[kk][0] = pack_bf16(p[0][0], p[0][1]);
        pa[kk][1] = pack_bf16(p[0][2], p[0][3]);
        pa[kk][2] = pack_bf16(p[1][0], p[1][1]);
        pa[kk][3] = pack_bf16(p[1][2], p[1][3]);
      }
      ps0 += __shfl_xor_sync(0xffffffffu, ps0, 1);
      ps0 += __shfl_xor_sync(0xffffffffu, ps0, 2);
      ps1 += __shfl_xor_sync(0xffffffffu, ps1, 1);
      ps1 += __shfl_xor_sync(0xffffffffu, ps1, 2);
      l0 = l0 * corr0 + ps0;
      l1 = l1 * corr1 + ps1;
      m0 = mn0;
      m1 = mn1;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        o[t][0] *= corr0;
        o[t][1] *= corr0;
        o[t][2] *= corr1;
        o[t][3] *= corr1;
      }
      {
        const int krow = (lane & 7) + (((lane >> 3) & 1) << 3);
        const int csel = lane >> 4;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const int key = kk * 16 + krow;
#pragma unroll
          for (int dt = 0; dt < NT / 2; ++dt) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(v_base + key * (D * 2) + (((2 * dt + csel) ^ (key & 7)) << 4), b0, b1, b2, b3);
            mma_bf16_16816(o[2 * dt], pa[kk], b0, b1);
            mma_bf16_16816(o[2 * dt + 1], pa[kk], b2, b3);
          }
        }
      }
    }
    __syncthreads();
  }

  const float inv0 = l0 > 0.f ? 1.0f / l0 : 0.f, inv1 = l1 > 0.f ? 1.0f / l1 : 0.f;
  if (r0 < n_tok) {
    __nv_bfloat16* dst = out + ((size_t)(q_start + tok0 + r0) * nh + head) * D;
#pragma unroll
    for (int t = 0; t < NT; ++t)
      *reinterpret_cast<uint32_t*>(dst + t * 8 + cpair) = pack_bf16(o[t][0] * inv0, o[t][1] * inv0);
  }
  if (r1 < n_tok) {
    __nv_bfloat16* dst = out + ((size_t)(q_start + tok0 + r1) * nh + head) * D;
#pragma unroll
    for (int t = 0; t < NT; ++t)
      *reinterpret_cast<uint32_t*>(dst + t * 8 + cpair) = pack_bf16(o[t][2] * inv1, o[t][3] * inv1);
  }
}

template <int D>
int launch_prefill_attention(const void* q, const void* kcache, const void* vcache, const int* block_table,
                             int bt_stride, const int* cu_q, const int* kv_before, const int* tile_seq,
                             const int* tile_tok0, int n_tiles, void* out, int nh, int nkv, int page_size,
                             float scale, int window, cudaStream_t stream) {
  const int smem = 2 * 2 * kPfBN * D * 2;
  auto kern = prefill_attention_bf16_kernel<D>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
  }
  const dim3 grid(n_tiles, nh);
  kern<<<grid, kPfWarps * 32, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kcache,
                                             (const __nv_bfloat16*)vcache, block_table, bt_stride, cu_q, kv_before,
                                             tile_seq, tile_tok0, (__nv_bfloat16*)out, nh, nkv, page_size,
                                             scale * 1.4426950408889634f, window);
  return launch_status();
}

}  // namespace tmk

// q, out [T, nh, D] bfloat16; caches [pages, page_size, nkv, D] bfloat16; tile_seq / tile_tok0 [n_tiles]:
// request and first token (within its portion) of each 64-token tile. Head sizes 64 and 128.
extern "C" int tm_prefill_attention_bf16(const void* q, const void* kcache, const void* vcache,
                                         const int* block_table, int bt_stride, const int* cu_q,
                                         const int* kv_before, const int* tile_seq, const int* tile_tok0,
                                         int n_tiles, void* out, int nh, int nkv, int D, int page_size, float scale,
                                         int window, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (nkv <= 0 || nh % nkv || page_size <= 0 || nh > 65535) return TM_ERR_UNSUPPORTED_SHAPE;
  if (D == 64)
    return tmk::launch_prefill_attention<64>(q, kcache, vcache, block_table, bt_stride, cu_q, kv_before, tile_seq,
                                             tile_tok0, n_tiles, out, nh, nkv, page_size, scale, window, stream);
  if (D == 128)
    return tmk::launch_prefill_attention<128>(q, kcache, vcache, block_table, bt_stride, cu_q, kv_before, tile_seq,
                                              tile_tok0, n_tiles, out, nh, nkv, page_size, scale, window, stream);
  return TM_ERR_UNSUPPORTED_SHAPE;
}
