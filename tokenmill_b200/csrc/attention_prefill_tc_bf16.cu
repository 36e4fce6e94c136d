// Causal attention of prompt portions over the paged cache on the 5th-generation tensor cores (tcgen05):
// bfloat16 in, scores and outputs accumulated in float32 in tensor memory, softmax in float32 registers.
// Head sizes 64 (blocks of 128 keys) and 128 (blocks of 64 keys: the same 112 KB of shared memory and 192
// columns of tensor memory either way). Semantics, work units and the merge of a row tile's key chunks are those of
// attention_prefill_bf16.cu (src/infer/model/layers.py:72-107, src/infer/kv/context.py:63-76); what differs
// is the row tile (128 rows of (token, head-in-group) instead of 64) and where the products run.
//
// One block of 256 threads per work unit (row tile, kv head, chunk of keys); threads r and r + 128 share row r,
// which is lane r of tensor memory: the first takes keys 0..63 of a block and output columns 0..31, the second
// the other halves, and they agree on the block's reference maximum through shared memory. Per block of 128 keys:
//   1. keys and values arrive by cp.async into 128-byte-swizzled tiles, two stages deep (8 neighbouring threads
//      bring the 8 16-byte pieces of a row; the rows' cache slots are looked up one tile ahead, stepping
//      through the pages with one division a tile);
//   2. one thread issues S = Q K^T (M 128 rows, N 128 keys, K 64) as 4 tcgen05.mma into 128 columns of tensor
//      memory and commits to an mbarrier;
//   3. every thread reads its half of its row of S back (tcgen05.ld), masks, takes the maximum, turns the scores into
//      probabilities (one fused multiply-add and exp2 each), keeps the running maximum and denominator, and
//      writes the probabilities as bfloat16 into a swizzled shared-memory tile; when the maximum moved, the
//      row's partial output in tensor memory is rescaled (tcgen05.ld / st);
//   4. one thread issues O += P V (M 128, N 64, K 128 keys; V is read as an MN-major operand straight from
//      its [key][dim] tile) as 8 tcgen05.mma into 64 more columns, commits, and issues the next block's
//      scores at once.
// The block that finishes a row tile last merges its chunks' partial results, which it brings into shared
// memory with bulk copies (one trip to the L2 for a pass of rows).
// With two blocks resident per SM one block's softmax overlaps the other's products. Every mbarrier wait is
// bounded: when one runs out the block raises the error word, skips its remaining work, frees its tensor
// memory and leaves (the host turns the word into an exception).
#include "tcgen05_util.cuh"
#include "mma_util.cuh"
#include "attention_merge.cuh"

namespace tmk {

constexpr int kTaBM = 128;                 // rows per work unit
// Head size 64 works on blocks of 128 keys, head size 128 on blocks of 64: either way a K or V stage is 16 KB,
// Q and P together 48 KB (16 + 32, or 32 + 16), S and O together 192 columns of tensor memory.
constexpr int kTaTile = 16384;             // a panel: 128 rows of 128 bytes (64 bfloat16)
constexpr int kTaXch = 512;                // the two halves' block maxima, bfloat16, [row][half]
constexpr int kTaSmem = kTaTile * 7 + 64 + kTaXch;   // Q, K x2, V x2, P; barriers and flags; maxima
constexpr int kTaThreads = 256;             // two threads per row: thread t and t + 128 share row t, 64 keys each
constexpr int kTaCols = 256;               // tensor-memory columns: S first, then O (192 of them used)

// Profiling aid: when set (tm_prefill_attention_tc_timing), the first thread of block 0's second warp (a warp
// that issues no products) stamps the nanosecond timer at the stations of its first units' key blocks: 8 stamps
// per key block, at most 64 blocks.
__device__ unsigned long long* g_ta_timing = nullptr;
// 2^x on the special-function unit, one instruction (exp2f adds range handling the softmax does not need:
// the argument is at most 0, and -inf gives 0).
__device__ __forceinline__ float ta_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void ta_stamp(int& at, int station) {
  if (g_ta_timing && blockIdx.x == 0 && threadIdx.x == 32 && at < 64) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_ta_timing[at * 8 + station] = t;
  }
}

template <int D>
__global__ void __launch_bounds__(kTaThreads, 2) prefill_attention_tc_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kcache,
    const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_table, int bt_stride,
    const int4* __restrict__ unit_rec, int n_units, int chunk_keys, float* __restrict__ part_acc,
    float* __restrict__ part_ml, int* __restrict__ tile_done, int* __restrict__ counters,
    __nv_bfloat16* __restrict__ out, int nh, int nkv, int page_size, float scale_log2, int window, int* error) {
  constexpr int BN = D == 64 ? 128 : 64;     // keys per block
  constexpr int QP = D / 64;                 // 64-column panels of a Q, K or V tile
  constexpr int PP = BN / 64;                // 64-key panels of the P tile
  constexpr int CPR = D / 8;                 // 16-byte pieces of a row
  constexpr int RPP = kTaThreads / CPR;      // rows the block copies per pass
  static_assert(D == 64 || D == 128, "head size 64 or 128");
  // All shared memory is the dynamic region (no static variables, no slack): two blocks then fit an SM. The
  // tiles need 1024-byte alignment (the swizzle pattern repeats every 1024 B); with nothing in front of it
  // the region starts aligned, which is checked below.
  extern __shared__ __align__(1024) unsigned char ta_smem_raw[];
  const uint32_t base = t5_smem(ta_smem_raw);
  // Tiles are stored as panels of [rows][128 bytes] with the 128-byte swizzle: Q [QP][128 rows], a K or V stage
  // [QP][BN rows] (16 KB either way), P [PP][128 rows].
  const uint32_t q_s = base, k_s = base + QP * kTaTile, v_s = k_s + 2 * kTaTile, p_s = v_s + 2 * kTaTile;
  constexpr uint32_t kPanelKV = BN * 128;    // bytes of one panel of a K or V stage
  unsigned char* tail = ta_smem_raw + 7 * kTaTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail);
  uint32_t& s_tmem_base = *reinterpret_cast<uint32_t*>(tail + 16);
  volatile int& s_abort = *reinterpret_cast<volatile int*>(tail + 20);
  int& s_ticket = *reinterpret_cast<int*>(tail + 24);
  __nv_bfloat16* xch = reinterpret_cast<__nv_bfloat16*>(tail + 64);
  const uint32_t bar_s = t5_smem(&bars[0]), bar_pv = t5_smem(&bars[1]), bar_m = t5_smem(&bars[4]);
  if (base & 1023u) {                        // (never seen; without it the products would read garbage)
    if (threadIdx.x == 0) atomicCAS(error, 0, 19);
    return;
  }
  const int tid = threadIdx.x, warp = tid >> 5;
  const int G = nh / nkv;
  const int total_units = n_units * nkv;

  if (tid == 0) {
    s_abort = 0;
    mbar_init(bar_s, 1);
    mbar_init(bar_pv, 1);
    mbar_init(bar_m, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(t5_smem(&s_tmem_base)), "r"(kTaCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  t5_fence_before();
  __syncthreads();
  t5_fence_after();
  // (Launched with programmatic dependent launch: the set-up above overlaps the end of the kernel in front, which
  // wrote the queries and the step's keys and values; nothing of a step is read before this wait.)
  pdl_launch_dependents();
  pdl_wait();
  // Thread t and thread t + 128 work on row t (tensor-memory lane t; a warp reaches the 32 lanes of its index
  // modulo 4): the first on keys 0..63 of a block and output columns 0..31, the second on the other halves.
  const int rt = tid & 127, half = tid >> 7;
  const uint32_t tmem_row = s_tmem_base + ((uint32_t)((warp & 3) * 32) << 16);   // this thread's lane, column 0
  const uint32_t tmem_s = s_tmem_base, tmem_o = s_tmem_base + BN;
  constexpr uint32_t idesc_qk = t5_idesc(kTaBM, BN, false), idesc_pv = t5_idesc(kTaBM, 64, true);
  uint32_t n_s = 0, n_pv = 0, n_m = 0;                // completed phases of the two barriers (uniform over the block)
  int stamp_at = 0;
  bool ok = true;

  while (ok) {
    __syncthreads();                         // the previous unit is done with shared memory and s_ticket
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
    const int n_rows = min(kTaBM, q_len * G - row0);
    if (n_rows <= 0) continue;
    const int p_min = before + row0 / G, p_max = before + (row0 + n_rows - 1) / G;
    const int j_lo = max(window > 0 ? max(0, p_min - window + 1) : 0, chunk * chunk_keys);
    const int j_hi = min(p_max, (chunk + 1) * chunk_keys - 1);
    const int* table = block_table + (size_t)s * bt_stride;
    const int kb_first = (j_lo / BN) * BN;
    const int n_blocks = j_lo > j_hi ? 0 : (j_hi - kb_first) / BN + 1;

    // This thread's row.
    const bool row_ok = rt < n_rows;
    const int row = row0 + (row_ok ? rt : 0);
    const int tok = row / G, g = row - tok * G;
    const size_t o_off = ((size_t)(q_start + tok) * nh + kvh * G + g) * D;
    const int p_row = row_ok ? before + tok : -1;
    const int lo_row = window > 0 ? max(0, p_row - window + 1) : 0;
    const uint32_t sw = (uint32_t)(rt & 7);

    // Loading a tile: CPR neighbouring threads bring the 16-byte pieces of one row (whole 128-byte lines), the
    // block RPP rows per pass, four passes for a stage of BN rows; piece c of row r goes to panel c / 8, place
    // ((c % 8) ^ (r % 8)) of the row. The cache slots of a tile's rows are looked up one tile ahead, so that no
    // copy waits for a table read.
    const int l_row = tid / CPR;                         // this thread's row within a pass
    const uint32_t l_piece = (uint32_t)(tid % CPR);
    const uint32_t l_panel = l_piece >> 3, l_chunk = l_piece & 7;
    int slots[4];                                        // cache slots of rows l_row + RPP i of the tile to load next
    auto look_up = [&](int kb) {                         // one division a tile: the rows step through the pages
      const int j0 = kb + l_row;
      int pg = j0 / page_size, off = j0 - pg * page_size;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = j0 + RPP * i;
        slots[i] = (j >= j_lo && j <= j_hi) ? table[pg] * page_size + off : -1;
        off += RPP;
        while (off >= page_size) { off -= page_size; ++pg; }
      }
    };
    auto load_kv = [&](int stage) {                      // uses `slots`, looked up for the tile to load
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = l_row + RPP * i;
        const bool has = slots[i] >= 0;
        const size_t src = has ? ((size_t)slots[i] * nkv + kvh) * D + l_piece * 8 : 0;
        const uint32_t off = l_panel * kPanelKV + (uint32_t)r * 128 + ((l_chunk ^ (uint32_t)(r & 7)) << 4);
        cp_async16(k_s + stage * kTaTile + off, kcache + src, has);        // rows without a key are zeros
        cp_async16(v_s + stage * kTaTile + off, vcache + src, has);
      }
    };
    auto issue_qk = [&](int stage) {                     // one thread: S = Q K^T, D / 16 steps of 16 columns
      t5_fence_after();
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        t5_mma(tmem_s, t5_desc(q_s + (ks >> 2) * kTaTile + (ks & 3) * 32),
               t5_desc(k_s + stage * kTaTile + (ks >> 2) * kPanelKV + (ks & 3) * 32), idesc_qk, ks ? 1u : 0u);
      t5_commit(bar_s);
    };
    if (n_blocks > 0) {
#pragma unroll
      for (int i = 0; i < kTaBM / RPP; ++i) {            // the queries: row r of the tile is row row0 + r
        const int r = l_row + RPP * i;
        const bool has = r < n_rows;
        const int qrow = row0 + (has ? r : 0), qtok = qrow / G, qg = qrow - qtok * G;
        cp_async16(q_s + l_panel * kTaTile + (uint32_t)r * 128 + ((l_chunk ^ (uint32_t)(r & 7)) << 4),
                   q + ((size_t)(q_start + qtok) * nh + kvh * G + qg) * D + l_piece * 8, has);
      }
      look_up(kb_first);
      load_kv(0);
      look_up(kb_first + BN);
    }
    cp_async_commit();
    cp_async_wait<0>();
    t5_fence_smem_writes();
    __syncthreads();                                     // the queries and block 0 have landed, for everyone
    if (tid == 0 && n_blocks > 0) issue_qk(0);

    float m_run = -INFINITY, l_run = 0.f;    // running maximum (scaled, log2 units) and denominator of the row
    for (int b = 0; b < n_blocks && ok; ++b) {
      const int kb = kb_first + b * BN, stage = b & 1;
      ta_stamp(stamp_at, 0);
      if (b > 0) {                           // the products before are done: P, the other stage and O are free
        ok = mbar_wait(bar_pv, n_pv & 1u, &s_abort, error, 11);
        ++n_pv;
        if (!ok) break;
      }
      ta_stamp(stamp_at, 1);
      if (b + 1 < n_blocks) {
        load_kv(stage ^ 1);
        look_up(kb + 2 * BN);
      }
      cp_async_commit();
      ta_stamp(stamp_at, 2);
      ok = mbar_wait(bar_s, n_s & 1u, &s_abort, error, 12);
      ++n_s;
      if (!ok) break;
      t5_fence_after();
      ta_stamp(stamp_at, 3);

      // This thread's BN / 2 scores of the row come into registers at once (all reads in flight, one wait).
      constexpr int SC = BN / 64;            // 32-column reads per thread
      const int col0 = half * (BN / 2);
      const int last = min(j_hi, p_row) - kb - col0, first = max(j_lo, lo_row) - kb - col0;   // visible: first..last
      float sv[SC][32];
#pragma unroll
      for (int c = 0; c < SC; ++c) t5_ld32(tmem_row + col0 + c * 32, sv[c]);
      t5_ld_wait();
      // Most blocks lie wholly inside every row's visible range: only the others pay for the mask.
      if (!(first <= 0 && last >= BN / 2 - 1)) {
#pragma unroll
        for (int c = 0; c < SC; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < first || c * 32 + i > last) sv[c][i] = -INFINITY;
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};     // four chains instead of one long one
#pragma unroll
      for (int c = 0; c < SC; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], sv[c][i]);
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // The row's two threads agree on one reference value: each leaves its own maximum, rounded UP to
      // bfloat16 (any value at or above the true maximum will do, as long as both use the same), and takes the
      // larger of the two.
      xch[rt * 2 + half] = __float2bfloat16_ru(mx * scale_log2);
      __syncthreads();
      const __nv_bfloat162 both = *reinterpret_cast<const __nv_bfloat162*>(xch + rt * 2);
      const float m_new = fmaxf(m_run, fmaxf(__bfloat162float(both.x), __bfloat162float(both.y)));
      const float mbase = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = m_new == -INFINITY ? 1.f : ta_exp2(m_run - m_new);
      // Probabilities, their sum, and this thread's part of the bfloat16 tile for the second product: key j of
      // the block lies in panel j / 64, piece (j % 64) / 8 of the row.
      float ps4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < SC; ++c) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          sv[c][i] = ta_exp2(fmaf(sv[c][i], scale_log2, -mbase));      // a masked score is -inf: 0
          ps4[i & 3] += sv[c][i];
        }
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          const uint32_t w0 = pack_bf16(sv[c][i], sv[c][i + 1]), w1 = pack_bf16(sv[c][i + 2], sv[c][i + 3]);
          const uint32_t w2 = pack_bf16(sv[c][i + 4], sv[c][i + 5]), w3 = pack_bf16(sv[c][i + 6], sv[c][i + 7]);
          const uint32_t j = (uint32_t)(col0 + c * 32 + i);
          const uint32_t row_s = p_s + (j >> 6) * kTaTile + rt * 128;
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(row_s + ((((j & 63) >> 3) ^ sw) << 4)), "r"(w0),
                       "r"(w1), "r"(w2), "r"(w3) : "memory");
        }
      }
      ta_stamp(stamp_at, 4);
      l_run = l_run * alpha + ((ps4[0] + ps4[1]) + (ps4[2] + ps4[3]));
      m_run = m_new;
      // The row's partial output follows the maximum (the first block of a unit starts it afresh).
      if (b > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
        for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {   // this thread's half of the columns
          float v[32];
          t5_ld32(tmem_row + BN + c0, v);
          t5_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] *= alpha;
          t5_st32(tmem_row + BN + c0, v);
        }
        t5_st_wait();
      }
      ta_stamp(stamp_at, 5);
      cp_async_wait<0>();                    // the next block's keys and values (asked for before the softmax)
      t5_fence_before();
      t5_fence_smem_writes();
      __syncthreads();                       // P is complete, S has been read, O rescaled, block b + 1 has landed
      ta_stamp(stamp_at, 6);
      if (tid == 0) {
        t5_fence_after();
        // O += P V, 64 output columns (one panel of V) at a time, BN / 16 steps of 16 keys each
#pragma unroll
        for (int dp = 0; dp < QP; ++dp)
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks)
            t5_mma(tmem_o + dp * 64, t5_desc(p_s + (ks >> 2) * kTaTile + (ks & 3) * 32),
                   t5_desc(v_s + stage * kTaTile + dp * kPanelKV + ks * 2048), idesc_pv, (b | ks) ? 1u : 0u);
        t5_commit(bar_pv);
        if (b + 1 < n_blocks) issue_qk(stage ^ 1);       // the next block's scores follow at once
      }
      ta_stamp(stamp_at, 7);
      ++stamp_at;
    }
    if (ok && n_blocks > 0) {
      ok = mbar_wait(bar_pv, n_pv & 1u, &s_abort, error, 13);
      ++n_pv;
    }
    if (!ok) break;
    t5_fence_after();

    // The row's result: normalised output when the tile has one chunk, else sums, maximum and denominator.
    // The row's two threads add up their halves of the denominator (through the P tile, free by now) and each
    // writes its 32 output columns. (Every thread takes part in the tensor-memory reads; only the stores depend
    // on the row being real.)
    {
      float* lx = reinterpret_cast<float*>(ta_smem_raw + (QP + 4) * kTaTile);      // [half][row], in the P tile
      lx[half * kTaBM + rt] = l_run;
      __syncthreads();
      const float l_row_sum = lx[rt] + lx[kTaBM + rt];
      const float inv = l_row_sum > 0.f ? 1.0f / l_row_sum : 0.f;
      const size_t prow = slot0 < 0 ? 0 : ((size_t)(slot0 + chunk) * nkv + kvh) * kTaBM + rt;
#pragma unroll 1
      for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
        float v[32];
        if (n_blocks > 0) {                  // uniform over the block
          t5_ld32(tmem_row + BN + c0, v);
          t5_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.f;
        }
        if (!row_ok) continue;
        if (slot0 < 0) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 o;
            o.x = pack_bf16(v[i] * inv, v[i + 1] * inv);
            o.y = pack_bf16(v[i + 2] * inv, v[i + 3] * inv);
            o.z = pack_bf16(v[i + 4] * inv, v[i + 5] * inv);
            o.w = pack_bf16(v[i + 6] * inv, v[i + 7] * inv);
            *reinterpret_cast<uint4*>(out + o_off + c0 + i) = o;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(part_acc + prow * D + c0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
      }
      if (row_ok && slot0 >= 0 && half == 0) *reinterpret_cast<float2*>(part_ml + prow * 2) = make_float2(m_run, l_row_sum);
    }
    t5_fence_before();
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
        // The chunks' partial results come into shared memory (all of it is free now) by bulk copies, as many
        // rows a pass as fit: one trip to the L2 for a pass instead of one for every few values. (Read piece by
        // piece into registers, a merge took longer than the unit's products.) Groups of 8 rows are copied
        // whole; a slot has 128 rows, so the rows past the tile's last exist and are not used.
        const int rows_fit = ((7 * kTaTile) / (n_chunks * (D * 4 + 8))) & ~7;
        if (rows_fit >= 8) {
          for (int r0 = 0; r0 < n_rows && ok; r0 += rows_fit) {
            const int rp = min(rows_fit, (n_rows - r0 + 7) & ~7), rows = min(rp, n_rows - r0);
            const uint32_t ml_s = base + (uint32_t)(n_chunks * rp * D * 4);
            __syncthreads();                 // the products and the pass before are done with shared memory
            if (tid == 0) {
              asm volatile("fence.proxy.async;" ::: "memory");
              mbar_expect_tx(bar_m, (uint32_t)(n_chunks * rp * (D * 4 + 8)));
              for (int c = 0; c < n_chunks; ++c) {
                const size_t prow = ((size_t)(slot0 + c) * nkv + kvh) * kTaBM + r0;
                bulk_load(base + (uint32_t)(c * rp * D * 4), part_acc + prow * D, (uint32_t)(rp * D * 4), bar_m);
                bulk_load(ml_s + (uint32_t)(c * rp * 8), part_ml + prow * 2, (uint32_t)(rp * 8), bar_m);
              }
            }
            ok = mbar_wait(bar_m, n_m & 1u, &s_abort, error, 14);
            ++n_m;
            if (!ok) break;
            // First the row's maximum over the chunks, then every chunk weighted by 2^(its maximum - that):
            // the weights do not depend on one another, so nothing waits for the exponential before it.
            const float* acc_f = reinterpret_cast<const float*>(ta_smem_raw);
            const float* ml_f = acc_f + n_chunks * rp * D;
            for (int idx = tid; idx < rows * (D / 4); idx += kTaThreads) {
              const int r = idx / (D / 4), piece = idx - r * (D / 4);
              float mx = -INFINITY;
              for (int c = 0; c < n_chunks; ++c) mx = fmaxf(mx, ml_f[(c * rp + r) * 2]);
              float lsum = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
              for (int c = 0; c < n_chunks; ++c) {
                const float2 ml = *reinterpret_cast<const float2*>(ml_f + (c * rp + r) * 2);
                const float4 pa = *reinterpret_cast<const float4*>(acc_f + ((c * rp + r) * (D / 4) + piece) * 4);
                const float w = ml.x == -INFINITY ? 0.f : ta_exp2(ml.x - mx);
                lsum += ml.y * w;
                acc[0] += pa.x * w;
                acc[1] += pa.y * w;
                acc[2] += pa.z * w;
                acc[3] += pa.w * w;
              }
              const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
              const int mrow = row0 + r0 + r, mtok = mrow / G, mg = mrow - mtok * G;
              uint2 ov;
              ov.x = pack_bf16(acc[0] * inv, acc[1] * inv);
              ov.y = pack_bf16(acc[2] * inv, acc[3] * inv);
              *reinterpret_cast<uint2*>(out + ((size_t)(q_start + mtok) * nh + kvh * G + mg) * D + piece * 4) = ov;
            }
          }
          if (!ok) break;
        } else {
          merge_tile_chunks<D, kTaBM, kTaThreads, 4>(part_acc, part_ml, slot0, n_chunks, nkv, kvh, n_rows, row0, G, q_start,
                                                     nh, out, tid);
        }
        if (tid == 0) tile_done[tile * nkv + kvh] = 0;
      }
    }
  }

  // Teardown: the block has left its loop (normally, or through a bounded wait). Copies of its own that may
  // still be on their way into shared memory are waited for, then the tensor memory goes back.
  cp_async_wait<0>();
  t5_fence_before();
  __syncthreads();
  if (warp == 0) {
    t5_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(s_tmem_base), "r"(kTaCols));
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

}  // namespace tmk

extern "C" int tm_prefill_attention_tc_timing(unsigned long long* stamps) {
  return (int)cudaMemcpyToSymbol(tmk::g_ta_timing, &stamps, sizeof(stamps));
}

// As tm_prefill_attention_bf16, for head sizes 64 and 128, with row tiles of 128 rows (the unit records and the
// partial-result slots are made for 128-row tiles: part_acc [slots * nkv, 128, D], part_ml [slots * nkv,
// 128, 2]). `error`: a device int that must be zero; a block whose wait runs out writes a non-zero code there
// instead of hanging.
extern "C" int tm_prefill_attention_tc_bf16(const void* q, const void* kcache, const void* vcache,
                                            const int* block_table, int bt_stride, const int* unit_rec, int n_units,
                                            int chunk_keys, float* part_acc, float* part_ml, int* tile_done,
                                            int* counters, void* out, int nh, int nkv, int D, int page_size,
                                            float scale, int window, int* error, cudaStream_t stream) {
  if (n_units <= 0) return 0;
  if ((D != 64 && D != 128) || nkv <= 0 || nh % nkv || page_size <= 0 || !counters || !error || chunk_keys <= 0 ||
      chunk_keys % 128 || !(scale > 0.f) || (reinterpret_cast<uintptr_t>(unit_rec) & 15))
    return TM_ERR_UNSUPPORTED_SHAPE;
  auto kern = D == 64 ? tmk::prefill_attention_tc_kernel<64> : tmk::prefill_attention_tc_kernel<128>;
  static int n_sm = 0;
  static bool prepared[2] = {false, false};
  if (!prepared[D == 128]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tmk::kTaSmem);
    if (e != cudaSuccess) return (int)e;
    // Two blocks of 112 KB per SM need nearly all of the SM's memory as shared memory.
    e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return (int)e;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    prepared[D == 128] = true;
  }
  // Two blocks per SM: by shared memory (2 x 112 KB), registers and tensor memory (2 x 256 columns) they fit,
  // although the occupancy query answers 1 here. Should an SM take only one at a time, the others start when
  // it leaves and find the ticket counter exhausted: slower, never wrong.
  const int blocks_per_sm = 2;
  const long long units = (long long)n_units * nkv;
  long long grid = (long long)n_sm * blocks_per_sm;
  if (grid > units) grid = units;
  return tmk::launch_pdl(kern, dim3((unsigned)grid), dim3(tmk::kTaThreads), (size_t)tmk::kTaSmem, stream,
                         (const __nv_bfloat16*)q, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_table,
                         bt_stride, reinterpret_cast<const int4*>(unit_rec), n_units, chunk_keys, part_acc, part_ml,
                         tile_done, counters, (__nv_bfloat16*)out, nh, nkv, page_size, scale * 1.4426950408889634f,
                         window, error);
}
