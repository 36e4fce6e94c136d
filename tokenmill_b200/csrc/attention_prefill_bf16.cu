// Causal attention of prompt portions over the paged cache on tensor cores (bfloat16 in, float32
// softmax and accumulate).
//
// Semantics as attention_paged.cu (src/infer/model/layers.py:72-107, src/infer/kv/context.py:63-76):
// the step's keys and values already sit in the cache; the query at absolute position p of a request
// reads that request's keys j <= p (and j > p - window if a window is set); query head h reads kv
// head h / G. Any mix of requests works (a decoded token is a portion of one).
//
// Work unit: 64 consecutive (token, head-in-group) rows of one request and one kv head (so the G query
// heads that share a kv head also share every key/value tile that is staged), times one CHUNK of keys cut
// at absolute multiples of `chunk_keys`. A causal prompt's last row tile sees 2T/64 times the keys of its
// first; without the cut the longest tile alone sets the kernel's duration while most SMs idle. Units are
// listed heaviest first by the host and handed out through an atomic ticket, so blocks that finish a short
// unit fetch the next one. A row tile with a single chunk writes its output itself; the others write
// unnormalised sums with their running maximum and denominator into per-(tile, chunk) slots, and the block
// that finishes a (tile, kv head) last merges them in chunk order. Chunks are anchored at absolute positions, so a row's
// sums run in the same order however the prompt was cut into portions. The ticket and a done-counter live
// in a two-int scratch; the last block to finish puts both back to 0.
//
// Per unit, keys stream through shared memory in blocks of 64 anchored at absolute positions 0, 64,
// 128, ... (cp.async ring; one page lookup per key row); each warp multiplies its rows with the whole
// block (ldmatrix + mma.sync.m16n8k16), keeps the online-softmax state in registers and adds P.V with V
// read through ldmatrix.trans. The anchoring makes a row's sums run in the same order however the
// prompt was cut into portions.
//
// This is the mma.sync ("legacy tensor core") formulation; it reaches a fraction of what a tcgen05
// kernel with the accumulators in tensor memory would, and is the stand-in until that kernel exists.
#include "mma_util.cuh"
#include "attention_merge.cuh"

namespace tmk {

constexpr int kPfBM = 64;        // rows per work unit
constexpr int kPfBN = 64;        // keys per stage

template <int D, int MT, int WARPS, int STAGES>   // MT 16-row tiles per warp; MT * WARPS * 16 == 64
__global__ void __launch_bounds__(WARPS * 32) prefill_attention_bf16_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kcache,
    const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_table, int bt_stride,
    const int4* __restrict__ unit_rec, int n_units, int chunk_keys, float* __restrict__ part_acc,
    float* __restrict__ part_ml, int* __restrict__ tile_done, int* __restrict__ counters,
    __nv_bfloat16* __restrict__ out, int nh, int nkv, int page_size, float scale_log2, int window) {
  static_assert(MT * WARPS * 16 == kPfBM, "a unit is 64 rows");
  constexpr int THREADS = WARPS * 32;
  constexpr int CH = D / 8;                    // 16-byte chunks per row
  constexpr int TPR = THREADS / kPfBN;         // threads that share one key row when loading
  constexpr int CPT = CH / TPR;                // chunks each of them copies
  constexpr int KS = D / 16;
  constexpr int NT = D / 8;
  constexpr int TILE_BYTES = kPfBN * D * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_ticket;
  const uint32_t smem_base = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = nh / nkv;
  const int cpair = (lane & 3) * 2;
  const int total_units = n_units * nkv;

  for (;;) {
    __syncthreads();                           // the previous unit is done with shared memory and s_ticket
    // (Asking for the next ticket a unit early would hide its round trip, but a block would then sit on a unit
    // while others have run out of work; measured slower.)
    if (tid == 0) s_ticket = atomicAdd(&counters[0], 1);
    __syncthreads();
    const int unit = s_ticket;
    if (unit >= total_units) break;
    const int ui = unit / nkv, kvh = unit - ui * nkv;
    // The unit's record: request, first row, chunk | chunks << 16, first slot; tile, first flat row of the
    // request, its tokens in this step, its tokens already in the cache.
    const int4 ra = __ldg(unit_rec + 2 * ui), rb = __ldg(unit_rec + 2 * ui + 1);
    const int s = ra.x, row0 = ra.y, chunk = ra.z & 0xffff, n_chunks = ra.z >> 16, slot0 = ra.w;
    const int tile = rb.x, q_start = rb.y, q_len = rb.z, before = rb.w;
    const int n_rows = min(kPfBM, q_len * G - row0);
    if (n_rows <= 0) continue;
    const int p_min = before + row0 / G, p_max = before + (row0 + n_rows - 1) / G;
    const int j_lo = max(window > 0 ? max(0, p_min - window + 1) : 0, chunk * chunk_keys);
    const int j_hi = min(p_max, (chunk + 1) * chunk_keys - 1);
    const int* table = block_table + (size_t)s * bt_stride;
    const bool empty = j_lo > j_hi;              // (a window that has passed the whole chunk) uniform over the block

    // Rows of this thread: tile mt, rows rr and rr + 8.
    uint32_t qa[MT][KS][4];
    int p_row[MT][2], lo_row[MT][2];
    size_t o_off[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int r = (warp * MT + mt) * 16 + (lane >> 2) + hh * 8;
        const bool ok = r < n_rows;
        const int row = row0 + (ok ? r : 0);
        const int tok = row / G, g = row - tok * G;
        o_off[mt][hh] = ((size_t)(q_start + tok) * nh + kvh * G + g) * D;
        p_row[mt][hh] = ok ? before + tok : -1;
        lo_row[mt][hh] = window > 0 ? max(0, p_row[mt][hh] - window + 1) : 0;
        const __nv_bfloat16* qr = q + o_off[mt][hh];
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const int c = ks * 16 + cpair;
          qa[mt][ks][hh] = ok ? *reinterpret_cast<const uint32_t*>(qr + c) : 0u;
          qa[mt][ks][2 + hh] = ok ? *reinterpret_cast<const uint32_t*>(qr + c + 8) : 0u;
        }
      }
    }
    // Visibility range of the warp's rows (consecutive rows: positions never decrease).
    const int w_first = min(warp * MT * 16, n_rows - 1), w_last = min(warp * MT * 16 + MT * 16 - 1, n_rows - 1);
    const bool warp_has_rows = warp * MT * 16 < n_rows;
    const int wp_lo = before + (row0 + w_first) / G, wp_hi = before + (row0 + w_last) / G;
    const int w_key_lo = window > 0 ? max(0, wp_lo - window + 1) : 0;        // first key any row sees
    const int w_full_lo = window > 0 ? max(0, wp_hi - window + 1) : 0;       // first key every row sees

    float m_run[MT][2], l_run[MT][2];
    float o[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      m_run[mt][0] = m_run[mt][1] = -INFINITY;
      l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
      for (int t = 0; t < NT; ++t) o[mt][t][0] = o[mt][t][1] = o[mt][t][2] = o[mt][t][3] = 0.f;
    }

    const int kb_first = (j_lo / kPfBN) * kPfBN;
    const int n_blocks = empty ? 0 : (j_hi - kb_first) / kPfBN + 1;

    auto load_block = [&](int stage, int kb) {
      const uint32_t k_dst = smem_base + stage * 2 * TILE_BYTES, v_dst = k_dst + TILE_BYTES;
      const int row = tid / TPR, part = tid - row * TPR;
      const int j = kb + row;
      const bool ok = j >= j_lo && j <= j_hi;
      size_t src = 0;
      if (ok) {
        const int page = table[j / page_size];
        src = (((size_t)page * page_size + (j % page_size)) * nkv + kvh) * D;
      }
#pragma unroll
      for (int i = 0; i < CPT; ++i) {
        const int c = part * CPT + i;
        const uint32_t off = row * (D * 2) + ((c ^ (row & 7)) << 4);
        cp_async16(k_dst + off, kcache + src + c * 8, ok);
        cp_async16(v_dst + off, vcache + src + c * 8, ok);
      }
    };

#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) {
      if (i < n_blocks) load_block(i, kb_first + i * kPfBN);
      cp_async_commit();
    }
    for (int b = 0; b < n_blocks; ++b) {
      cp_async_wait<STAGES - 2>();             // block b has landed (this thread's copies)
      __syncthreads();                         // ... everyone's; and block b - 1 is fully consumed
      {
        const int nb = b + STAGES - 1;
        if (nb < n_blocks) load_block(nb % STAGES, kb_first + nb * kPfBN);
        cp_async_commit();
      }
      const int kb = kb_first + b * kPfBN;
      const int stage = b % STAGES;
      if (!warp_has_rows || kb > wp_hi || kb + kPfBN - 1 < w_key_lo) continue;   // nothing visible to this warp

      const uint32_t k_base = smem_base + stage * 2 * TILE_BYTES, v_base = k_base + TILE_BYTES;
      float sc[MT][8][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int t = 0; t < 8; ++t) sc[mt][t][0] = sc[mt][t][1] = sc[mt][t][2] = sc[mt][t][3] = 0.f;
      {
        const int krow = (lane & 7) + ((lane >> 4) << 3);
        const int csel = (lane >> 3) & 1;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const int key = kk * 16 + krow;
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(k_base + key * (D * 2) + (((2 * ks + csel) ^ (key & 7)) << 4), b0, b1, b2, b3);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              mma_bf16_16816(sc[mt][2 * kk], qa[mt][ks], b0, b1);
              mma_bf16_16816(sc[mt][2 * kk + 1], qa[mt][ks], b2, b3);
            }
          }
        }
      }
      // Every key of the block visible to every row of the warp: no mask needed.
      const bool need_mask = kb + kPfBN - 1 > wp_lo || kb < w_full_lo;
      uint32_t pa[MT][4][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
        for (int t = 0; t < 8; ++t)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = kb + t * 8 + cpair + e;
            bool ok0 = true, ok1 = true;
            if (need_mask) {
              ok0 = j <= p_row[mt][0] && j >= lo_row[mt][0];
              ok1 = j <= p_row[mt][1] && j >= lo_row[mt][1];
            }
            if (!ok0) sc[mt][t][e] = -INFINITY;
            if (!ok1) sc[mt][t][2 + e] = -INFINITY;
            tmax0 = fmaxf(tmax0, sc[mt][t][e]);
            tmax1 = fmaxf(tmax1, sc[mt][t][2 + e]);
          }
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
        // The maximum is taken over the raw scores and scaled once (the scale is positive); the exponent's
        // argument is then one fused multiply-add per score.
        const float mn0 = fmaxf(m_run[mt][0], tmax0 * scale_log2), mn1 = fmaxf(m_run[mt][1], tmax1 * scale_log2);
        const float corr0 = mn0 == -INFINITY ? 1.f : exp2f(m_run[mt][0] - mn0);
        const float corr1 = mn1 == -INFINITY ? 1.f : exp2f(m_run[mt][1] - mn1);
        const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          float p[2][4];
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              p[h][e] = exp2f(fmaf(sc[mt][2 * kk + h][e], scale_log2, -base0));          // masked entries are -inf: 0
              p[h][2 + e] = exp2f(fmaf(sc[mt][2 * kk + h][2 + e], scale_log2, -base1));
              ps0 += p[h][e];
              ps1 += p[h][2 + e];
            }
          pa[mt][kk][0] = pack_bf16(p[0][0], p[0][1]);
          pa[mt][kk][1] = pack_bf16(p[0][2], p[0][3]);
          pa[mt][kk][2] = pack_bf16(p[1][0], p[1][1]);
          pa[mt][kk][3] = pack_bf16(p[1][2], p[1][3]);
        }
        ps0 += __shfl_xor_sync(0xffffffffu, ps0, 1);
        ps0 += __shfl_xor_sync(0xffffffffu, ps0, 2);
        ps1 += __shfl_xor_sync(0xffffffffu, ps1, 1);
        ps1 += __shfl_xor_sync(0xffffffffu, ps1, 2);
        l_run[mt][0] = l_run[mt][0] * corr0 + ps0;
        l_run[mt][1] = l_run[mt][1] * corr1 + ps1;
        m_run[mt][0] = mn0;
        m_run[mt][1] = mn1;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          o[mt][t][0] *= corr0;
          o[mt][t][1] *= corr0;
          o[mt][t][2] *= corr1;
          o[mt][t][3] *= corr1;
        }
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
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              mma_bf16_16816(o[mt][2 * dt], pa[mt][kk], b0, b1);
              mma_bf16_16816(o[mt][2 * dt + 1], pa[mt][kk], b2, b3);
            }
          }
        }
      }
    }
    cp_async_wait<0>();

#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        if (p_row[mt][hh] < 0) continue;
        const float l = l_run[mt][hh];
        if (slot0 < 0) {                         // the tile's only chunk: normalise and write the output
          const float inv = l > 0.f ? 1.0f / l : 0.f;
          __nv_bfloat16* dst = out + o_off[mt][hh];
#pragma unroll
          for (int t = 0; t < NT; ++t)
            *reinterpret_cast<uint32_t*>(dst + t * 8 + cpair) =
                pack_bf16(o[mt][t][2 * hh] * inv, o[mt][t][2 * hh + 1] * inv);
        } else {                                 // one of several: sums, maximum (log2 units) and denominator
          const int r = (warp * MT + mt) * 16 + (lane >> 2) + hh * 8;
          const size_t prow = ((size_t)(slot0 + chunk) * nkv + kvh) * kPfBM + r;
          float* dst = part_acc + prow * D;
#pragma unroll
          for (int t = 0; t < NT; ++t)
            *reinterpret_cast<float2*>(dst + t * 8 + cpair) = make_float2(o[mt][t][2 * hh], o[mt][t][2 * hh + 1]);
          if ((lane & 3) == 0) *reinterpret_cast<float2*>(part_ml + prow * 2) = make_float2(m_run[mt][hh], l);
        }
      }
    if (slot0 >= 0) {
      // The block that finishes a (row tile, kv head) last merges its chunks, in chunk order, each weighted by
      // 2^(its maximum - the maximum so far); rows a chunk had no key for carry a maximum of -inf and a zero
      // denominator and drop out. The arrival counter is left at zero for the next launch.
      __threadfence();
      __syncthreads();
      if (tid == 0) s_ticket = atomicAdd(&tile_done[tile * nkv + kvh], 1);
      __syncthreads();
      if (s_ticket == n_chunks - 1) {
        __threadfence();
        merge_tile_chunks<D, kPfBM, THREADS, 4>(part_acc, part_ml, slot0, n_chunks, nkv, kvh, n_rows, row0, G, q_start, nh,
                                                  out, tid);
        if (tid == 0) tile_done[tile * nkv + kvh] = 0;
      }
    }
  }

  // The last block to leave puts the ticket and the done-counter back to zero for the next launch.
  if (tid == 0) {
    __threadfence();
    const int done = atomicAdd(&counters[1], 1);
    if (done == (int)gridDim.x - 1) {
      counters[0] = 0;
      counters[1] = 0;
      __threadfence();
    }
  }
}

template <int D, int MT, int WARPS, int STAGES>
int launch_prefill_attention(const void* q, const void* kcache, const void* vcache, const int* block_table,
                             int bt_stride, const int* unit_rec, int n_units, int chunk_keys, float* part_acc,
                             float* part_ml, int* tile_done, int* counters, void* out, int nh, int nkv,
                             int page_size, float scale, int window, cudaStream_t stream) {
  const int smem = STAGES * 2 * kPfBN * D * 2;
  auto kern = prefill_attention_bf16_kernel<D, MT, WARPS, STAGES>;
  static int blocks_per_sm = 0, n_sm = 0;
  if (smem + 1024 > 48 * 1024) {   // the kernel's static shared memory counts against the 48 KB default too
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
  }
  if (blocks_per_sm == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks_per_sm, kern, WARPS * 32, smem);
    if (e != cudaSuccess || blocks_per_sm < 1) blocks_per_sm = 1;
  }
  const long long units = (long long)n_units * nkv;
  long long grid = (long long)n_sm * blocks_per_sm;
  if (grid > units) grid = units;
  kern<<<(int)grid, WARPS * 32, smem, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_table, bt_stride,
      reinterpret_cast<const int4*>(unit_rec), n_units, chunk_keys, part_acc, part_ml, tile_done, counters,
      (__nv_bfloat16*)out, nh, nkv, page_size, scale * 1.4426950408889634f, window);
  return launch_status();
}

}  // namespace tmk

// q, out [T, nh, D] bfloat16; caches [pages, page_size, nkv, D] bfloat16. unit_rec [n_units, 8] ints, 16-byte
// aligned, heaviest first: request, first (token, head-in-group) row of the 64-row tile, key chunk | chunks of
// the tile << 16 (keys chunk * chunk_keys ...; chunk_keys a multiple of 64), first partial slot of the tile
// (-1: single chunk), tile index, first flat row of the request, its tokens in this step, its tokens already in
// the cache. part_acc [slots * nkv, 64, D] and part_ml [slots * nkv, 64, 2] float32, tile_done [tiles * nkv]
// ints that are zero before the first launch and left zero (all three may be null when no tile has several
// chunks). counters: two ints that are zero before the first launch (the kernel leaves them zero). The scale
// must be positive. Head sizes 64 and 128.
extern "C" int tm_prefill_attention_bf16(const void* q, const void* kcache, const void* vcache,
                                         const int* block_table, int bt_stride, const int* unit_rec, int n_units,
                                         int chunk_keys, float* part_acc, float* part_ml, int* tile_done,
                                         int* counters, void* out, int nh, int nkv, int D, int page_size,
                                         float scale, int window, cudaStream_t stream) {
  if (n_units <= 0) return 0;
  if (nkv <= 0 || nh % nkv || page_size <= 0 || !counters || chunk_keys <= 0 || chunk_keys % tmk::kPfBN ||
      !(scale > 0.f) || (reinterpret_cast<uintptr_t>(unit_rec) & 15))
    return TM_ERR_UNSUPPORTED_SHAPE;
  if (D == 64)
    return tmk::launch_prefill_attention<64, 1, 4, 3>(q, kcache, vcache, block_table, bt_stride, unit_rec, n_units,
                                                      chunk_keys, part_acc, part_ml, tile_done, counters, out, nh,
                                                      nkv, page_size, scale, window, stream);
  if (D == 128)
    return tmk::launch_prefill_attention<128, 1, 4, 2>(q, kcache, vcache, block_table, bt_stride, unit_rec, n_units,
                                                       chunk_keys, part_acc, part_ml, tile_done, counters, out, nh,
                                                       nkv, page_size, scale, window, stream);
  return TM_ERR_UNSUPPORTED_SHAPE;
}
