// Decode attention over the paged cache, driven by a list of work units, with the keys and values brought in by
// the tensor memory accelerator (bfloat16, head size 64 or 128, pages of 8, 16, 32 or 64 tokens). The arithmetic
// is that of src/infer/model/layers.py:100-124 over the cache of src/infer/kv/context.py:77-79: every query row
// sees the keys up to its own position (and not older than the window), softmax in 32-bit.
//
// The host cuts each request's keys into UNITS of whole 64-key stages (parts/attention_plan.py decode_units: as many
// units as keep every block of the grid busy for the same time, however the step's requests differ in length) and
// writes them as records {request, first stage, end stage, part | parts << 16}. The grid is persistent: block b
// takes work items b, b + gridDim.x, ... of the list, an item being (unit, kv head). A block is two warps.
//
//   * The PRODUCER warp walks the block's items and fills a ring of stages with `cp.async.bulk.tensor`: a page's
//     keys of one kv head are one box of a 2-D tensor map over the cache ([slots, kv_heads * head_dim], box = page
//     rows x 64 columns, 128-byte swizzle: the layout ldmatrix reads without bank conflicts), one lane per box.
//     It only waits for a ring slot to be given back, so it runs ahead of the arithmetic, across item borders.
//   * The CONSUMER warp takes the stages in order: scores of 16 query rows against 64 keys on the tensor cores
//     (mma.sync m16n8k16), an online softmax, the values; at an item's end its state is the unit's PARTIAL, written
//     straight from the registers. The block that writes the last partial of a (request, kv head) merges them in
//     part order. (One consumer per ring: a ring slot is always read by the same warp, so the parity it waits for
//     cannot be mistaken for that of a fill it has not seen.)
//
// Every wait is bounded (tcgen05_util.cuh mbar_wait): a block that gives up raises the error word, waits (bounded)
// for the copies it asked for and leaves. A stage's rows beyond the unit's keys are filled from the nearest page
// inside the unit (their scores are masked; what matters is that they hold finite numbers: the pool starts zeroed
// and only finite values are ever written).
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <vector>

#include "attention_decode_core.cuh"
#include "tcgen05_util.cuh"

namespace tmk {

constexpr int kTdMaxPages = 256;           // pages of one unit: at most 32 stages of 64 keys in pages of 8
constexpr int kTdMaxStages = 32;           // stages of one unit (attention_plan.py DECODE_MAX_UNIT_STAGES)
template <int D> __host__ __device__ constexpr int td_stage_bytes() { return 2 * kDecBN * D * 2; }   // K and V tiles
template <int D> __host__ __device__ constexpr int td_stages() { return D == 64 ? 3 : 2; }
template <int D> __host__ __device__ constexpr int td_blocks_per_sm() { return D == 64 ? 4 : 3; }

__device__ __forceinline__ void td_tma_load(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

// Where 16-byte piece `chunk` of key row `key` lies in a tile of 64 keys: halves of 64 columns one after the other,
// rows of 128 bytes, pieces XOR-swizzled by the row (what the 128-byte swizzle of the tensor map writes).
__device__ __forceinline__ uint32_t td_tile_addr(uint32_t base, int key, int chunk) {
  return base + (uint32_t)(chunk >> 3) * (kDecBN * 128) + (uint32_t)key * 128 + (uint32_t)(((chunk & 7) ^ (key & 7)) << 4);
}

// 2^x by the hardware's approximation (2 ulp; the argument is at most 0, and -inf gives 0).
__device__ __forceinline__ float td_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Profiling aid: when set (tm_decode_attention_units_timing), block 0 writes the global timer at its stations,
// 8 a work item for its first 7 items ([64] unsigned 64-bit): 0 entry, 1 set up; then from 2 + 8 * item:
// queries loaded, first stage landed, last stage done, partial written, merged (if it was the last); producer:
// first copy asked for, last copy asked for; consumer again: counted.
__device__ unsigned long long* g_td_timing = nullptr;

__device__ __forceinline__ void td_stamp(unsigned long long* at, int station) {
  if (at && station < 64) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    at[station] = t;
  }
}

// What a work item covers, worked out the same way by both warps.
struct TdItem {
  int s, kvh, part, parts;
  int q_start, n_rows, before, p_max;
  int j_lo, j_hi;            // first and last key of the item
  int kb_first, n_stages;    // first key of its first stage, stages (0: nothing to do)
};

__device__ __forceinline__ TdItem td_item(const int4* __restrict__ units, int w, const int* __restrict__ cu_q,
                                          const int* __restrict__ kv_before, int nh, int nkv, int window) {
  TdItem it;
  const int4 rec = units[w / nkv];
  it.s = rec.x;
  it.kvh = w % nkv;
  it.part = rec.w & 0xffff;
  it.parts = rec.w >> 16;
  it.q_start = cu_q[it.s];
  const int q_len = cu_q[it.s + 1] - it.q_start;
  const int G = nh / nkv;
  it.before = kv_before[it.s];
  it.n_rows = min(q_len * G, 16);
  it.p_max = it.before + (it.n_rows - 1) / G;
  const int lo = window > 0 ? max(0, it.before - window + 1) : 0;
  it.j_lo = max(lo, rec.y * kDecBN);
  it.j_hi = min(it.p_max, rec.z * kDecBN - 1);
  it.kb_first = (it.j_lo / kDecBN) * kDecBN;
  it.n_stages = (it.n_rows <= 0 || it.j_lo > it.j_hi) ? 0 : (it.j_hi - it.kb_first) / kDecBN + 1;
  return it;
}

// The merge of a (request, kv head)'s partial results, by one warp. A lane owns 4 columns of up to SLOTS rows at
// a time and takes the parts PP at a time, in part order: the loads of a pass (2 x SLOTS x PP a lane, 32 in both
// shapes used) are all asked for before the first is used, so a pass costs one trip to the L2. Few rows (heads
// of 64 in groups of up to 8: two rows share a warp's 32 lanes) take 4 parts a pass, more rows 2.
template <int D, int SLOTS, int PP>
__device__ __forceinline__ void td_merge_parts(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                               __nv_bfloat16* __restrict__ out, const TdItem& it, int n_rows, int G,
                                               int nh, int max_parts, int lane) {
  constexpr int GROUPS = D / 4, LANE_ROWS = 32 / GROUPS;
  const int d = (lane % GROUPS) * 4;
  for (int rb = 0; rb < n_rows; rb += SLOTS * LANE_ROWS) {
    int orow[SLOTS];
    float mx[SLOTS], lsum[SLOTS], acc[SLOTS][4];
#pragma unroll
    for (int i = 0; i < SLOTS; ++i) {
      const int r = rb + i * LANE_ROWS + lane / GROUPS;
      orow[i] = r < n_rows ? (it.q_start + r / G) * nh + it.kvh * G + r % G : -1;
      mx[i] = -INFINITY;
      lsum[i] = 0.f;
      acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    }
    for (int z0 = 0; z0 < it.parts; z0 += PP) {
      float2 ml[SLOTS][PP];
      float4 pv[SLOTS][PP];
#pragma unroll
      for (int i = 0; i < SLOTS; ++i)
#pragma unroll
        for (int u = 0; u < PP; ++u) {
          const bool have = orow[i] >= 0 && z0 + u < it.parts;
          const size_t at = (size_t)max(orow[i], 0) * max_parts + min(z0 + u, it.parts - 1);
          ml[i][u] = have ? __ldcg(reinterpret_cast<const float2*>(part_ml + at * 2)) : make_float2(-INFINITY, 0.f);
          pv[i][u] = have ? __ldcg(reinterpret_cast<const float4*>(part_acc + at * D + d)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
      for (int u = 0; u < PP; ++u)
#pragma unroll
        for (int i = 0; i < SLOTS; ++i) {
          const float m_new = fmaxf(mx[i], ml[i][u].x);
          const float sub = m_new == -INFINITY ? 0.f : m_new;      // (no key yet on either side: both weigh 0)
          const float keep = td_exp2(mx[i] - sub), wgt = td_exp2(ml[i][u].x - sub);
          lsum[i] = lsum[i] * keep + ml[i][u].y * wgt;
          acc[i][0] = acc[i][0] * keep + pv[i][u].x * wgt;
          acc[i][1] = acc[i][1] * keep + pv[i][u].y * wgt;
          acc[i][2] = acc[i][2] * keep + pv[i][u].z * wgt;
          acc[i][3] = acc[i][3] * keep + pv[i][u].w * wgt;
          mx[i] = m_new;
        }
    }
#pragma unroll
    for (int i = 0; i < SLOTS; ++i)
      if (orow[i] >= 0) {
        const float inv = lsum[i] > 0.f ? 1.0f / lsum[i] : 0.f;
        uint2 ov;
        ov.x = pack_bf16(acc[i][0] * inv, acc[i][1] * inv);
        ov.y = pack_bf16(acc[i][2] * inv, acc[i][3] * inv);
        *reinterpret_cast<uint2*>(out + (size_t)orow[i] * D + d) = ov;
      }
  }
}

// What the kernel needs to finish the q/k/v projection itself (ROPE variant): the raw product of the step's tokens,
// the bias, the rotation tables and where each token's key and value go. Then no kernel stands between the
// projection and the attention: the consumer warp adds the bias and rotates its query rows while it loads them
// (rotate-half, src/infer/model/layers.py:60-64, in the arithmetic of rope_cache.cu), and the item whose unit holds
// a new token's position computes that token's key and value for its kv head, writes them to the cache and puts
// them into the stage it has just received (where the copy brought the slot's old content).
struct TdRope {
  const __nv_bfloat16* qkv;      // [T, (nh + 2 nkv) D]
  const float* bias;             // [(nh + 2 nkv) D] or null
  const int* positions;          // [T]
  const float* cos_t;            // [n_pos, D / 2]
  const float* sin_t;
  const int* slot_map;           // [T] cache slot of each token (negative: not written)
  __nv_bfloat16* kcache;
  __nv_bfloat16* vcache;
  int n_pos;
};

__device__ __forceinline__ int td_rope_position(int pos, int n_pos, int* error) {
  if (pos >= 0 && pos < n_pos) return pos;
  if (error) atomicCAS(error, 0, 31);          // never read outside the tables; tell the host
  return pos < 0 ? 0 : n_pos - 1;
}

__device__ __forceinline__ float2 td_bf16x2(uint32_t v) {
  __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&v);
  return __bfloat1622float2(h);
}

template <int D, bool ROPE>
__global__ void __launch_bounds__(64) decode_attention_units_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
    const __nv_bfloat16* __restrict__ q, const int* __restrict__ block_table, int bt_stride,
    const int* __restrict__ cu_q, const int* __restrict__ kv_before, const int4* __restrict__ units,
    const int* __restrict__ n_work_ptr, int max_work, float* __restrict__ part_acc, float* __restrict__ part_ml,
    __nv_bfloat16* __restrict__ out, int* __restrict__ done, int nh, int nkv, int page_size, float scale_log2,
    int window, int max_parts, int* __restrict__ error, const TdRope rp) {
  constexpr int KS = D / 16, NT = D / 8, NS = td_stages<D>(), STAGE = td_stage_bytes<D>(), TILE = kDecBN * D * 2;
  extern __shared__ __align__(1024) unsigned char td_raw[];
  __shared__ __align__(8) uint64_t s_full[NS], s_empty[NS];
  __shared__ int s_pages[kTdMaxPages];       // (the producer's own: the pages of the item it is filling)
  __shared__ int s_abort;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t ring = (t5_smem(td_raw) + 1023u) & ~1023u;
  pdl_launch_dependents();
  // (The unit list, the requests' lengths and the block table are the step's inputs, copied before its first
  // kernel: they and the older keys and values may be read before the kernel in front of this one has finished.)
  unsigned long long* stamps = (g_td_timing && blockIdx.x == 0 && lane == 0) ? g_td_timing : nullptr;
  td_stamp(warp == 0 ? stamps : nullptr, 0);
  const int n_work = min(*n_work_ptr, max_work);
  const int G = nh / nkv;
  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < NS; ++i) {
      mbar_init(t5_smem(&s_full[i]), 1);
      mbar_init(t5_smem(&s_empty[i]), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  td_stamp(warp == 0 ? stamps : nullptr, 1);

  bool ok = true;
  int issued = 0;                            // (producer) stages asked for so far, over all items
  if (warp == 1) {
    // ---- producer: the copies of a stage are spread over the lanes: lane = (box, half head, K or V), at most 8 x 2 x 2 ----
    const int page_log = 31 - __clz(page_size);                 // (page sizes are powers of two)
    const int rows = min(page_size, kDecBN);                    // rows of a box
    const int boxes = kDecBN / rows;
    constexpr int HALVES = D / 64;
    const int my_box = lane / (2 * HALVES), my_half = (lane / 2) % HALVES, my_v = lane & 1;
    const bool copies = my_box < boxes;
    const CUtensorMap* my_map = my_v ? &map_v : &map_k;
    const uint32_t my_off = (uint32_t)my_v * TILE + (uint32_t)my_half * (kDecBN * 128) + (uint32_t)(my_box * rows) * 128;
    bool waited = false;
    int item = 0;
    for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++item) {
      const TdItem it = td_item(units, w, cu_q, kv_before, nh, nkv, window);
      if (it.n_stages <= 0) continue;
      if (it.n_stages > kTdMaxStages) {      // (a plan this kernel cannot hold: say so and stop)
        if (lane == 0) atomicCAS(error, 0, 32);
        s_abort = 1;
        ok = false;
        break;
      }
      const int page0 = it.kb_first >> page_log;
      const int n_pages = (it.j_hi >> page_log) - page0 + 1;
      __syncwarp();                          // the copies of the item before have been asked for: its pages may go
      for (int i = lane; i < n_pages; i += 32) s_pages[i] = block_table[(size_t)it.s * bt_stride + page0 + i];
      __syncwarp();
      const int j_first = it.j_lo & ~(rows - 1), j_last = it.j_hi & ~(rows - 1);
      const int x = it.kvh * D + my_half * 64;
      for (int k = 0; k < it.n_stages; ++k) {
        const int slot = issued % NS;
        if (issued >= NS) {
          ok = mbar_wait(t5_smem(&s_empty[slot]), (uint32_t)(issued / NS - 1) & 1u, &s_abort, error, 34);
          if (!ok) break;
        }
        const int kb = it.kb_first + k * kDecBN;
        if (!ROPE && !waited && kb + kDecBN > it.before) {      // keys of the step's own tokens: written by the
          pdl_wait();                                           // kernel in front of this one (with ROPE: by the
          waited = true;                                        // consumer, into the stage itself)
        }
        const uint32_t bar = t5_smem(&s_full[slot]);
        if (k == 0 && item < 7) td_stamp(stamps, 2 + 8 * item + 5);
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)STAGE);
        __syncwarp();
        if (copies) {
          const int j0 = min(max(kb + my_box * rows, j_first), j_last);
          const int y = (s_pages[(j0 >> page_log) - page0] << page_log) + (j0 & (page_size - 1));
          td_tma_load(ring + (uint32_t)slot * STAGE + my_off, my_map, x, y, bar);
        }
        ++issued;
      }
      if (item < 7) td_stamp(stamps, 2 + 8 * item + 6);
    }
    pdl_wait();                              // (every thread of the chain waits before it exits)
  } else {
    // ---- consumer: the stages in order, 64 keys at a time, one online softmax per item ----
    pdl_wait();                              // the queries come from the kernel in front of this one
    const int r0 = lane >> 2, r1 = r0 + 8;   // the two tile rows this thread's accumulators belong to
    const int cpair = (lane & 3) * 2;
    const int k_key = (lane & 7) + ((lane >> 4) << 3), k_sel = (lane >> 3) & 1;     // ldmatrix rows: keys, not transposed
    const int v_key = (lane & 7) + (((lane >> 3) & 1) << 3), v_sel = lane >> 4;     // and transposed, for the values
    int taken = 0;                           // stages read so far, over all items
    int item = 0;
    for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++item) {
      const TdItem it = td_item(units, w, cu_q, kv_before, nh, nkv, window);
      if (it.n_stages <= 0) continue;
      if (it.n_stages > kTdMaxStages) break;
      const int n_rows = it.n_rows, before = it.before;
      uint32_t qa[KS][4];                    // query fragments straight from global memory (rows beyond n_rows are zero)
      if constexpr (!ROPE) {
        const __nv_bfloat16* qr0 = nullptr;
        const __nv_bfloat16* qr1 = nullptr;
        if (r0 < n_rows) qr0 = q + ((size_t)(it.q_start + r0 / G) * nh + it.kvh * G + r0 % G) * D;
        if (r1 < n_rows) qr1 = q + ((size_t)(it.q_start + r1 / G) * nh + it.kvh * G + r1 % G) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const int c = ks * 16 + cpair;
          qa[ks][0] = qr0 ? __ldcg(reinterpret_cast<const unsigned int*>(qr0 + c)) : 0u;
          qa[ks][1] = qr1 ? __ldcg(reinterpret_cast<const unsigned int*>(qr1 + c)) : 0u;
          qa[ks][2] = qr0 ? __ldcg(reinterpret_cast<const unsigned int*>(qr0 + c + 8)) : 0u;
          qa[ks][3] = qr1 ? __ldcg(reinterpret_cast<const unsigned int*>(qr1 + c + 8)) : 0u;
        }
      } else {
        // The raw projection's rows: bias added and rotated here. A lane's elements of the first half of a head
        // (steps ks < KS / 2) and their partners of the second half (ks + KS / 2) are both its own.
        constexpr int half_d = D / 2;
        const int width = (nh + 2 * nkv) * D;
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
          const int r = hrow ? r1 : r0;
          if (r >= n_rows) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) qa[ks][hrow] = qa[ks][2 + hrow] = 0u;
            continue;
          }
          const int tok = it.q_start + r / G, head = it.kvh * G + r % G;
          const __nv_bfloat16* src = rp.qkv + (size_t)tok * width + head * D;
          const float* bsrc = rp.bias ? rp.bias + head * D : nullptr;
          const int pos = td_rope_position(rp.positions[tok], rp.n_pos, error);
          const float* cs = rp.cos_t + (size_t)pos * half_d;
          const float* sn = rp.sin_t + (size_t)pos * half_d;
#pragma unroll
          for (int ks = 0; ks < KS / 2; ++ks)
#pragma unroll
            for (int part = 0; part < 2; ++part) {           // elements c, c + 1 and c + 8, c + 9
              const int c = ks * 16 + cpair + part * 8;
              float2 x1 = td_bf16x2(__ldcg(reinterpret_cast<const unsigned int*>(src + c)));
              float2 x2 = td_bf16x2(__ldcg(reinterpret_cast<const unsigned int*>(src + c + half_d)));
              if (bsrc) {
                const float2 b1 = __ldg(reinterpret_cast<const float2*>(bsrc + c));
                const float2 b2 = __ldg(reinterpret_cast<const float2*>(bsrc + c + half_d));
                x1.x += b1.x; x1.y += b1.y; x2.x += b2.x; x2.y += b2.y;
              }
              const float2 cc = __ldg(reinterpret_cast<const float2*>(cs + c));
              const float2 ss = __ldg(reinterpret_cast<const float2*>(sn + c));
              const float o1x = __fadd_rn(__fmul_rn(x1.x, cc.x), __fmul_rn(-x2.x, ss.x));
              const float o1y = __fadd_rn(__fmul_rn(x1.y, cc.y), __fmul_rn(-x2.y, ss.y));
              const float o2x = __fadd_rn(__fmul_rn(x2.x, cc.x), __fmul_rn(x1.x, ss.x));
              const float o2y = __fadd_rn(__fmul_rn(x2.y, cc.y), __fmul_rn(x1.y, ss.y));
              qa[ks][hrow + 2 * part] = pack_bf16(o1x, o1y);
              qa[ks + KS / 2][hrow + 2 * part] = pack_bf16(o2x, o2y);
            }
        }
      }
      if (item < 7) td_stamp(stamps, 2 + 8 * item);
      const int p_r0 = r0 < n_rows ? before + r0 / G : -1, p_r1 = r1 < n_rows ? before + r1 / G : -1;
      const int lo_r0 = window > 0 ? max(0, p_r0 - window + 1) : 0, lo_r1 = window > 0 ? max(0, p_r1 - window + 1) : 0;
      const int lo_max = window > 0 ? max(0, it.p_max - window + 1) : 0;
      float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // running max (log2 units) and sum per row
      float o[NT][4];
#pragma unroll
      for (int t = 0; t < NT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;

      for (int b = 0; b < it.n_stages; ++b) {
        const int kb = it.kb_first + b * kDecBN;
        const int slot = taken % NS;
        ok = mbar_wait(t5_smem(&s_full[slot]), (uint32_t)(taken / NS) & 1u, &s_abort, error, 33);
        if (!ok) break;
        if (b == 0 && item < 7) td_stamp(stamps, 2 + 8 * item + 1);
        const uint32_t k_base = ring + (uint32_t)slot * STAGE, v_base = k_base + TILE;
        if constexpr (ROPE) {
          // The step's own tokens whose positions lie in this stage (and in this item's keys): their key and value
          // for this kv head, finished here, written to the cache and into the stage.
          const int q_tokens = (n_rows + G - 1) / G;
          const int t_lo = max(0, max(kb, it.j_lo) - before), t_hi = min(q_tokens - 1, min(kb + kDecBN - 1, it.j_hi) - before);
          if (t_lo <= t_hi) {
            constexpr int half_d = D / 2;
            const int width = (nh + 2 * nkv) * D;
            unsigned char* stage_ptr = td_raw + (k_base - t5_smem(td_raw));
            for (int tt = t_lo; tt <= t_hi; ++tt) {
              const int tok = it.q_start + tt, row = before + tt - kb;
              const int pos = td_rope_position(rp.positions[tok], rp.n_pos, error);
              const int cache_slot = rp.slot_map ? rp.slot_map[tok] : -1;
              const __nv_bfloat16* ksrc = rp.qkv + (size_t)tok * width + (nh + it.kvh) * D;
              const __nv_bfloat16* vsrc = ksrc + nkv * D;
              const float* kb_bias = rp.bias ? rp.bias + (nh + it.kvh) * D : nullptr;
              const float* vb_bias = rp.bias ? kb_bias + nkv * D : nullptr;
              for (int i = lane; i < half_d; i += 32) {
                float k1 = __bfloat162float(ksrc[i]), k2 = __bfloat162float(ksrc[i + half_d]);
                float v1 = __bfloat162float(vsrc[i]), v2 = __bfloat162float(vsrc[i + half_d]);
                if (kb_bias) {
                  k1 += kb_bias[i]; k2 += kb_bias[i + half_d];
                  v1 += vb_bias[i]; v2 += vb_bias[i + half_d];
                }
                const float c = rp.cos_t[(size_t)pos * half_d + i], sv = rp.sin_t[(size_t)pos * half_d + i];
                const __nv_bfloat16 ok1 = __float2bfloat16_rn(__fadd_rn(__fmul_rn(k1, c), __fmul_rn(-k2, sv)));
                const __nv_bfloat16 ok2 = __float2bfloat16_rn(__fadd_rn(__fmul_rn(k2, c), __fmul_rn(k1, sv)));
                const __nv_bfloat16 ov1 = __float2bfloat16_rn(v1), ov2 = __float2bfloat16_rn(v2);
                if (cache_slot >= 0) {
                  const size_t at = ((size_t)cache_slot * nkv + it.kvh) * D;
                  rp.kcache[at + i] = ok1; rp.kcache[at + i + half_d] = ok2;
                  rp.vcache[at + i] = ov1; rp.vcache[at + i + half_d] = ov2;
                }
                // element d of key row `row`: piece d / 8 of the row, swizzled as the copies write it
                auto put = [&](uint32_t tile_off, int d, __nv_bfloat16 val) {
                  const uint32_t off = td_tile_addr(tile_off, row, d >> 3) + (uint32_t)(d & 7) * 2;
                  *reinterpret_cast<__nv_bfloat16*>(stage_ptr + off) = val;
                };
                put(0u, i, ok1); put(0u, i + half_d, ok2);
                put((uint32_t)TILE, i, ov1); put((uint32_t)TILE, i + half_d, ov2);
              }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // these writes come before the slot's next copies
            __syncwarp();
          }
        }
        float sc[8][4];
#pragma unroll
        for (int t = 0; t < 8; ++t) sc[t][0] = sc[t][1] = sc[t][2] = sc[t][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(td_tile_addr(k_base, g * 16 + k_key, 2 * ks + k_sel), b0, b1, b2, b3);
            mma_bf16_16816(sc[2 * g], qa[ks], b0, b1);
            mma_bf16_16816(sc[2 * g + 1], qa[ks], b2, b3);
          }
        // Scale into log2 units; mask where the stage reaches beyond the keys a row may see (uniform over the warp;
        // rows beyond n_rows are never written out).
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
        if (kb >= it.j_lo && kb >= lo_max && kb + kDecBN - 1 <= min(it.j_hi, before)) {
#pragma unroll
          for (int t = 0; t < 8; ++t) {
#pragma unroll
            for (int e = 0; e < 4; ++e) sc[t][e] *= scale_log2;
            tmax0 = fmaxf(tmax0, fmaxf(sc[t][0], sc[t][1]));
            tmax1 = fmaxf(tmax1, fmaxf(sc[t][2], sc[t][3]));
          }
        } else {
#pragma unroll
          for (int t = 0; t < 8; ++t)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int j = kb + t * 8 + cpair + e;
              const bool in = j >= it.j_lo && j <= it.j_hi;
              sc[t][e] = (in && j <= p_r0 && j >= lo_r0) ? sc[t][e] * scale_log2 : -INFINITY;
              sc[t][2 + e] = (in && j <= p_r1 && j >= lo_r1) ? sc[t][2 + e] * scale_log2 : -INFINITY;
              tmax0 = fmaxf(tmax0, sc[t][e]);
              tmax1 = fmaxf(tmax1, sc[t][2 + e]);
            }
        }
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
        const float mn0 = fmaxf(m0, tmax0), mn1 = fmaxf(m1, tmax1);
        // (A row that has seen no key yet subtracts 0 instead of -inf: its scores are all -inf and come out as 0.)
        const float sub0 = mn0 == -INFINITY ? 0.f : mn0, sub1 = mn1 == -INFINITY ? 0.f : mn1;
        const float corr0 = td_exp2(m0 - sub0), corr1 = td_exp2(m1 - sub1);
        float ps0 = 0.f, ps1 = 0.f;
        uint32_t pa[4][4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float p[2][4];
#pragma unroll
          for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              p[t][e] = td_exp2(sc[2 * g + t][e] - sub0);
              p[t][2 + e] = td_exp2(sc[2 * g + t][2 + e] - sub1);
              ps0 += p[t][e];
              ps1 += p[t][2 + e];
            }
          pa[g][0] = pack_bf16(p[0][0], p[0][1]);
          pa[g][1] = pack_bf16(p[0][2], p[0][3]);
          pa[g][2] = pack_bf16(p[1][0], p[1][1]);
          pa[g][3] = pack_bf16(p[1][2], p[1][3]);
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
#pragma unroll
        for (int g = 0; g < 4; ++g)
#pragma unroll
          for (int dt = 0; dt < NT / 2; ++dt) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(td_tile_addr(v_base, g * 16 + v_key, 2 * dt + v_sel), b0, b1, b2, b3);
            mma_bf16_16816(o[2 * dt], pa[g], b0, b1);
            mma_bf16_16816(o[2 * dt + 1], pa[g], b2, b3);
          }
        __syncwarp();                                                   // the warp has read the stage
        if (lane == 0) mbar_arrive(t5_smem(&s_empty[slot]));
        ++taken;
      }
      if (!ok) break;
      if (item < 7) td_stamp(stamps, 2 + 8 * item + 2);

      if (it.parts == 1) {
        // The request's only unit: its state is the result.
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = half ? r1 : r0;
          if (r < n_rows) {
            const size_t orow = (size_t)(it.q_start + r / G) * nh + it.kvh * G + r % G;
            const float l = half ? l1 : l0;
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            __nv_bfloat16* dst = out + orow * D + cpair;
#pragma unroll
            for (int t = 0; t < NT; ++t)
              *reinterpret_cast<uint32_t*>(dst + t * 8) = pack_bf16(o[t][2 * half] * inv, o[t][2 * half + 1] * inv);
          }
        }
        if (item < 7) td_stamp(stamps, 2 + 8 * item + 3);
      } else {
        // The item's state is the unit's partial (max in log2 units, sum, unnormalised values).
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = half ? r1 : r0;
          if (r < n_rows) {
            const size_t orow = (size_t)(it.q_start + r / G) * nh + it.kvh * G + r % G;
            float* dst = part_acc + (orow * max_parts + it.part) * D + cpair;
#pragma unroll
            for (int t = 0; t < NT; ++t)
              *reinterpret_cast<float2*>(dst + t * 8) = make_float2(o[t][2 * half], o[t][2 * half + 1]);
            if ((lane & 3) == 0)
              *reinterpret_cast<float2*>(part_ml + (orow * max_parts + it.part) * 2) =
                  make_float2(half ? m1 : m0, half ? l1 : l0);
          }
        }
        if (item < 7) td_stamp(stamps, 2 + 8 * item + 3);
        // The last of a (request, kv head)'s units to finish merges them, in part order.
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) last = atomicAdd(&done[it.s * nkv + it.kvh], 1) == it.parts - 1;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (item < 7) td_stamp(stamps, 2 + 8 * item + 7);
        if (last) {
          __threadfence();
          if ((n_rows + (32 / (D / 4)) - 1) / (32 / (D / 4)) <= 4)
            td_merge_parts<D, 4, 4>(part_acc, part_ml, out, it, n_rows, G, nh, max_parts, lane);
          else
            td_merge_parts<D, 8, 2>(part_acc, part_ml, out, it, n_rows, G, nh, max_parts, lane);
          if (lane == 0) done[it.s * nkv + it.kvh] = 0;
        }
      }
      if (item < 7) td_stamp(stamps, 2 + 8 * item + 4);
    }
  }
  __syncthreads();                           // both warps: all copies have been asked for, all stages read, or one gave up
  if (s_abort && warp == 1 && lane == 0) {
    // Leaving early: give the copies still on their way into this block's shared memory a bounded chance to land
    // (the producer knows which fills it asked for: the last one of each slot, by its parity).
    for (int k = max(0, issued - NS); k < issued; ++k)
      for (uint32_t spin = 0; spin < (1u << 18) && !mbar_try(t5_smem(&s_full[k % NS]), (uint32_t)(k / NS) & 1u); ++spin)
        __nanosleep(64);
  }
}

// --- host -----------------------------------------------------------------------------------------------------

using TdEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static TdEncodeFn td_encode_fn() {
  static TdEncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TdEncodeFn>(p);
  }
  return fn;
}

struct TdMapKey {
  const void* base;
  long long slots;
  int page_size, nkv, D;
  bool operator==(const TdMapKey& o) const {
    return base == o.base && slots == o.slots && page_size == o.page_size && nkv == o.nkv && D == o.D;
  }
};

// The tensor map of one cache tensor ([slots, nkv * D] bfloat16, boxes of min(page, 64) rows x 64 columns, 128-byte
// swizzle). Encoding takes microseconds on the host, and a layer's cache never moves: maps are kept by address.
static bool td_map_for(const void* base, long long slots, int page_size, int nkv, int D, CUtensorMap* out) {
  static std::mutex mu;
  static std::vector<std::pair<TdMapKey, CUtensorMap>> maps;
  const TdMapKey key{base, slots, page_size, nkv, D};
  std::lock_guard<std::mutex> lock(mu);
  for (auto& kv : maps)
    if (kv.first == key) {
      *out = kv.second;
      return true;
    }
  TdEncodeFn fn = td_encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)nkv * D, (cuuint64_t)slots};
  const cuuint64_t strides[1] = {(cuuint64_t)nkv * D * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)(page_size < kDecBN ? page_size : kDecBN)};
  const cuuint32_t elem[2] = {1u, 1u};
  CUtensorMap m;
  if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (maps.size() >= 4096) maps.clear();     // (engines come and go in one process: do not grow without bound)
  maps.emplace_back(key, m);
  *out = m;
  return true;
}

template <int D, bool ROPE>
int launch_decode_attention_units(const CUtensorMap& mk, const CUtensorMap& mv, const void* q, const int* block_table,
                                  int bt_stride, const int* cu_q, const int* kv_before, const int* units,
                                  const int* n_work, int max_work, int grid_blocks, float* part_acc, float* part_ml,
                                  void* out, int* done, int nh, int nkv, int page_size, float scale, int window,
                                  int max_parts, int* error, const TdRope& rp, cudaStream_t stream) {
  const int smem = td_stages<D>() * td_stage_bytes<D>() + 1024;
  auto kern = decode_attention_units_kernel<D, ROPE>;
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    set = true;
  }
  return launch_pdl(kern, dim3(grid_blocks), dim3(64), (size_t)smem, stream, mk, mv, (const __nv_bfloat16*)q,
                    block_table, bt_stride, cu_q, kv_before, reinterpret_cast<const int4*>(units), n_work, max_work,
                    part_acc, part_ml, (__nv_bfloat16*)out, done, nh, nkv, page_size,
                    scale * 1.4426950408889634f, window, max_parts, error, rp);
}

static int decode_attention_units(const void* q, const TdRope& rp, bool rope, const void* kcache, const void* vcache,
                                  long long n_pages, const int* block_table, int bt_stride, const int* cu_q,
                                  const int* kv_before, const int* units, const int* n_work, int max_work,
                                  int grid_blocks, float* part_acc, float* part_ml, void* out, int* done, int nh,
                                  int nkv, int D, int page_size, float scale, int window, int max_parts, int* error,
                                  cudaStream_t stream) {
  if (max_work <= 0 || grid_blocks <= 0) return 0;
  if (nkv <= 0 || nh % nkv || nh / nkv > 16 || n_pages <= 0) return TM_ERR_UNSUPPORTED_SHAPE;
  if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return TM_ERR_UNSUPPORTED_SHAPE;
  if (max_parts <= 0 || max_parts > 0x7fff) return TM_ERR_UNSUPPORTED_SHAPE;
  if (D != 64 && D != 128) return TM_ERR_UNSUPPORTED_SHAPE;
  if ((reinterpret_cast<uintptr_t>(kcache) | reinterpret_cast<uintptr_t>(vcache) | reinterpret_cast<uintptr_t>(units)) & 15)
    return TM_ERR_UNSUPPORTED_SHAPE;
  if (!part_acc || !part_ml || !done || !out || !error || !units || !n_work) return TM_ERR_SCRATCH_TOO_SMALL;
  CUtensorMap mk, mv;
  if (!td_map_for(kcache, n_pages * page_size, page_size, nkv, D, &mk) ||
      !td_map_for(vcache, n_pages * page_size, page_size, nkv, D, &mv))
    return 90006;
#define TD_UNITS_ARGS mk, mv, q, block_table, bt_stride, cu_q, kv_before, units, n_work, max_work, grid_blocks, part_acc, \
                      part_ml, out, done, nh, nkv, page_size, scale, window, max_parts, error, rp, stream
  if (D == 64) return rope ? launch_decode_attention_units<64, true>(TD_UNITS_ARGS) : launch_decode_attention_units<64, false>(TD_UNITS_ARGS);
  return rope ? launch_decode_attention_units<128, true>(TD_UNITS_ARGS) : launch_decode_attention_units<128, false>(TD_UNITS_ARGS);
#undef TD_UNITS_ARGS
}

}  // namespace tmk

// Where block 0 writes its stations (device memory, [64] unsigned 64-bit; null turns it off).
extern "C" int tm_decode_attention_units_timing(unsigned long long* stamps) {
  return (int)cudaMemcpyToSymbol(tmk::g_td_timing, &stamps, sizeof(stamps));
}

// Blocks of the persistent grid that are resident at once on a chip of `sm_count` multiprocessors: what the host's
// plan of units should fill evenly.
extern "C" int tm_decode_attention_units_slots(int D, int sm_count) {
  return sm_count * (D == 64 ? tmk::td_blocks_per_sm<64>() : tmk::td_blocks_per_sm<128>());
}

// Decode attention by a list of units. q, out: [T, nh, D] bfloat16; caches [n_pages, page_size, nkv, D] bfloat16
// (16-byte aligned, for the tensor maps); block_table [n_seqs, bt_stride]; cu_q [n_seqs + 1]; kv_before [n_seqs];
// units: int32 [.., 4] records {request, first stage, end stage, part | parts << 16} (16-byte aligned), of which
// *n_work / nkv are valid (n_work on the device, at most max_work); every request with query rows has `parts` units
// that together cover its keys, part numbers 0 .. parts - 1 < max_parts, at most 32 stages a unit. part_acc
// [T * nh * max_parts * D] and part_ml [T * nh * max_parts * 2] float32 scratch; done: n_seqs * nkv zeroed counters
// (left zeroed). Every request brings at most 16 / (nh / nkv) query tokens. `error` (required) receives 32 for a
// plan the kernel cannot hold, 33 / 34 for a wait that ran out. Page sizes 8, 16, 32, 64; head sizes 64 and 128;
// anything else returns TM_ERR_UNSUPPORTED_SHAPE.
extern "C" int tm_decode_attention_units_bf16(const void* q, const void* kcache, const void* vcache, long long n_pages,
                                              const int* block_table, int bt_stride, const int* cu_q,
                                              const int* kv_before, const int* units, const int* n_work, int max_work,
                                              int grid_blocks, float* part_acc, float* part_ml, void* out, int* done,
                                              int nh, int nkv, int D, int page_size, float scale, int window,
                                              int max_parts, int* error, cudaStream_t stream) {
  if (!q) return TM_ERR_SCRATCH_TOO_SMALL;
  return tmk::decode_attention_units(q, tmk::TdRope{}, false, kcache, vcache, n_pages, block_table, bt_stride, cu_q,
                                     kv_before, units, n_work, max_work, grid_blocks, part_acc, part_ml, out, done, nh,
                                     nkv, D, page_size, scale, window, max_parts, error, stream);
}

// The same straight from the raw q/k/v product of the step's tokens: qkv [T, (nh + 2 nkv) D] bfloat16 (bias [..]
// float32 or null not yet added, nothing rotated), positions [T], rotate-half tables cos / sin [n_pos, D / 2]
// float32, slot_map [T] (the cache slot of each token's key and value; negative: not written). The kernel adds the
// bias, rotates the query rows as it loads them, and finishes, writes to the cache and uses each new token's key
// and value itself: the kernel that would do that between the product and the attention (rope_cache.cu) is not
// launched. A position outside the tables is clamped and raises error code 31.
extern "C" int tm_decode_attention_units_rope_bf16(const void* qkv, const float* bias, const int* positions,
                                                   const float* cos_t, const float* sin_t, int n_pos,
                                                   const int* slot_map, void* kcache, void* vcache, long long n_pages,
                                                   const int* block_table, int bt_stride, const int* cu_q,
                                                   const int* kv_before, const int* units, const int* n_work,
                                                   int max_work, int grid_blocks, float* part_acc, float* part_ml,
                                                   void* out, int* done, int nh, int nkv, int D, int page_size,
                                                   float scale, int window, int max_parts, int* error,
                                                   cudaStream_t stream) {
  if (!qkv || !positions || !cos_t || !sin_t || n_pos <= 0) return TM_ERR_SCRATCH_TOO_SMALL;
  if ((reinterpret_cast<uintptr_t>(qkv) & 3) || (reinterpret_cast<uintptr_t>(bias) & 7) ||
      (reinterpret_cast<uintptr_t>(cos_t) & 7) || (reinterpret_cast<uintptr_t>(sin_t) & 7))
    return TM_ERR_UNSUPPORTED_SHAPE;
  tmk::TdRope rp{};
  rp.qkv = (const __nv_bfloat16*)qkv; rp.bias = bias; rp.positions = positions; rp.cos_t = cos_t; rp.sin_t = sin_t;
  rp.slot_map = slot_map; rp.kcache = (__nv_bfloat16*)kcache; rp.vcache = (__nv_bfloat16*)vcache; rp.n_pos = n_pos;
  return tmk::decode_attention_units(nullptr, rp, true, kcache, vcache, n_pages, block_table, bt_stride, cu_q, kv_before,
                                     units, n_work, max_work, grid_blocks, part_acc, part_ml, out, done, nh, nkv, D,
                                     page_size, scale, window, max_parts, error, stream);
}
