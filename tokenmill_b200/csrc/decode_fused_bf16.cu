// One kernel for a whole decode step (bfloat16, at most 16 tokens): every layer's norm, QKV projection with
// bias / rotation / cache write, split-key attention, output projection, norm, gate/up projection with
// SwiGLU, down projection, and the final norm of the wanted rows. The output matrix and the sampling stay
// separate launches.
//
// Why: at these sizes each of the roughly 200 kernels of a decode step runs for a few microseconds and is
// bound by dependent memory round trips, not by bandwidth; launching them one after the other (even from a
// captured graph, even with programmatic dependent launch) costs more than the work. Here one persistent
// block per SM walks through the phases of all layers; the phases are separated by a grid-wide barrier
// (one atomic arrival counter in global memory, monotone within a launch), so a phase boundary costs an L2
// round trip instead of a launch and a drain.
//
// Phases per layer (the formulas are those of the separate kernels, which stay the reference for tests:
// norm.cu, gemm_skinny_bf16.cu, attention_decode_bf16.cu; reference model: src/infer/model/qwen2.py:13-23,
// src/infer/model/layers.py:127-164):
//   A  every block computes x = residual (+ the previous layer's down-projection output, or the embedding
//      rows for the first layer) for all tokens, norms it into shared memory, and block r writes row r of the
//      new residual; then the blocks share the QKV weight rows (8 + 8 partner rows per unit, K cut across the
//      8 warps), add bias, rotate, and write q and the cache slots.
//   B  attention units (request, kv head, key split), two per block at a time (4 warps each); the unit that
//      finishes a (request, kv head) last merges the splits in index order and writes the head outputs.
//   C  output projection from the staged head outputs to a 32-bit [T, H] buffer.
//   D  as A with the attention branch and the second norm, then gate/up + SwiGLU into a [T, I] buffer.
//   E  down projection to a 32-bit [T, H] buffer, which the next layer's phase A (or the final norm) adds.
// Data written by other blocks is read with L2-level loads (ld.global.cg / cp.async.cg), since L1 is not
// coherent across SMs within a launch; weights are read-only.
//
// The barrier's spin is bounded: a block that waits too long raises the error word, stops working and
// leaves; the others run into the same limit and leave too. The launch is cooperative, so all blocks are
// resident together. The arrival counter is put back to zero by the last block to leave.
#include "mma_util.cuh"

namespace tmk {

constexpr int kFuThreads = 256;
constexpr int kFuWarps = 8;
constexpr uint32_t kFuSpinLimit = 1u << 22;

struct FusedLayer {
  const float* ln1_w;
  // the four matrices in the packed layout described at fu_packed()
  const __nv_bfloat16* w_qkv;      // [(nh + 2 nkv) D, H]
  const float* b_qkv;              // [(nh + 2 nkv) D] or null
  __nv_bfloat16* kcache;           // [pages, page_size, nkv, D]
  __nv_bfloat16* vcache;
  const __nv_bfloat16* w_o;        // [H, nh D]
  const float* ln2_w;
  const __nv_bfloat16* w_gu;       // [2 I, H]
  const __nv_bfloat16* w_down;     // [H, I]
};

struct FusedArgs {
  const FusedLayer* layers;
  int n_layers;
  int H, nh, nkv, D, I;
  float eps1, eps2, eps_f, scale_log2;
  int window;
  const __nv_bfloat16* embedding;
  const float* final_ln_w;
  const float* cos_t;
  const float* sin_t;
  int n_pos;
  // the step
  const int* token_ids;
  const int* positions;
  const int* slot_map;
  const int* block_table;
  int bt_stride;
  const int* cu_q;
  const int* kv_before;
  const int* want_rows;
  int T, S, n_want, page_size, split_keys, max_splits;
  // workspaces
  float* resid;                    // [T, H] the 32-bit residual stream; the projections add into it
  __nv_bfloat16* q;                // [T, nh, D]
  float* part_acc;                 // [T nh, max_splits, D]
  float* part_ml;                  // [T nh, max_splits, 2]
  __nv_bfloat16* attn;             // [T, nh D]
  __nv_bfloat16* act;              // [T, I]
  int* attn_count;                 // [S, nkv], zero between launches
  unsigned* bar;                   // [1] arrival counter, zero between launches
  int* error;
  __nv_bfloat16* hidden_out;       // [n_want, H]
  int smem_bytes;                  // dynamic shared memory of the launch (set by the launcher)
  unsigned long long* timing;      // null, or [n_layers * 16 + 1] nanosecond stamps written by block 0 (profiling aid)
};

enum : int { FU_QKV = 0, FU_SWIGLU = 1, FU_ADD_RESID = 2 };

__device__ __forceinline__ void fu_stamp(const FusedArgs& a, int slot) {
  if (a.timing && blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    a.timing[slot] = t;
  }
}

__device__ __forceinline__ uint4 fu_ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void fu_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Ask for `bytes` at `base` to be brought into L2 (no completion to wait for): the whole grid shares the
// range in 4 KB pieces, one instruction per piece. The weights of the phase after next stream from HBM
// while this phase computes and the grid barriers are crossed, so the products read L2.
__device__ __forceinline__ void fu_prefetch_l2(const void* base, size_t bytes) {
  if (!base || (reinterpret_cast<uintptr_t>(base) & 15)) return;
  constexpr size_t kPiece = 4096;
  const size_t n_pieces = (bytes + kPiece - 1) / kPiece;
  for (size_t p = blockIdx.x + (size_t)threadIdx.x * gridDim.x; p < n_pieces; p += (size_t)gridDim.x * kFuThreads) {
    const size_t off = p * kPiece;
    const uint32_t sz = (uint32_t)((bytes - off < kPiece ? bytes - off : kPiece) & ~(size_t)15);
    if (sz) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(static_cast<const char*>(base) + off), "r"(sz) : "memory");
  }
}

// The weights are read in a packed copy (made once, when the decoder is set up): for every group of 8 rows
// and every chunk of 32 columns, the 32 lanes' 16-byte pieces lie one after the other in lane order (lane
// 4 g + t holds row g, columns 8 t .. 8 t + 7 of the chunk; rows and columns beyond the matrix are zeros).
// A warp's load is then 512 contiguous bytes. With the plain row-major matrix the same load touches 8 rows
// with 64 bytes each, which the memory system serves at a quarter of the rate.
constexpr int kFuChunkElems = 32 * 8;
__device__ __forceinline__ const __nv_bfloat16* fu_packed(const __nv_bfloat16* W, int row0, int n_chunks, int lane) {
  return W + ((size_t)(row0 >> 3) * n_chunks * 32 + lane) * 8;
}

__device__ __forceinline__ int fu_row_bytes(int K) {
  const int kpad = (K + 31) / 32 * 32;
  return kpad * 2 + ((64 - (kpad * 2) % 128) + 128) % 128;   // 64 mod 128: conflict-free fragment reads
}

// Grid-wide barrier number `k` (0-based) of this launch, in two halves: arrive (this block's writes are
// published) and wait (every block's are visible). Work that does not depend on other blocks may stand
// between them. The wait returns false when it ran out.
__device__ __forceinline__ void fu_grid_arrive(const FusedArgs& a) {
  __syncthreads();
  // Release-arrive at device scope: the block's writes (ordered before by the block barrier above) are
  // visible to every block that sees the counter reach the target.
  if (threadIdx.x == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(a.bar) : "memory");
}
__device__ __forceinline__ bool fu_grid_wait(const FusedArgs& a, unsigned& k, int* s_ok) {
  if (threadIdx.x == 0) {
    const unsigned target = (k + 1) * gridDim.x;
    uint32_t spins = 0;
    for (;;) {
      unsigned seen;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(a.bar) : "memory");
      if (seen >= target) break;
      if (++spins > kFuSpinLimit) {
        atomicCAS(a.error, 0, 100 + (int)k);
        *s_ok = 0;
        break;
      }
      if (spins > 64) __nanosleep(20);
    }
  }
  ++k;
  __syncthreads();
  return *s_ok != 0;
}
__device__ __forceinline__ bool fu_grid_sync(const FusedArgs& a, unsigned& k, int* s_ok) {
  fu_grid_arrive(a);
  return fu_grid_wait(a, k, s_ok);
}

// x[r] = source row r (the embedding row in the first layer, else the residual stream), for all T rows; the
// normed row goes to shared memory in bfloat16. In the first layer block r also writes x[r] to the residual
// stream. One warp per row. A lane's loads of a pass are issued together (up to kNormBatch groups of 4
// elements in flight) so that a row costs a couple of L2 round trips, not one per element; rows wider than
// a batch take several batches and are read twice.
constexpr int kNormBatch = 8;     // float4 groups per lane per batch: 8 * 32 * 4 = 1024 elements

__device__ __forceinline__ void fu_load_x4(const __nv_bfloat16* erow, const float* rrow, int i, float (&x)[4]) {
  if (erow) {
    load4<__nv_bfloat16>(erow + i, x);
  } else {
    const float4 r4 = __ldcg(reinterpret_cast<const float4*>(rrow + i));
    x[0] = r4.x; x[1] = r4.y; x[2] = r4.z; x[3] = r4.w;
  }
}

__device__ __noinline__ void fu_norm_rows(int T, int H, const __nv_bfloat16* embedding, const int* token_ids,
                                          float* resid, const float* ln_w, float eps, unsigned char* xs,
                                          int row_bytes) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n4 = H / 4;                                    // float4 groups per row (H is a multiple of 8)
  for (int r = warp; r < T; r += kFuWarps) {               // rows beyond T feed accumulator rows nobody reads
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(xs + (size_t)r * row_bytes);
    const __nv_bfloat16* erow = embedding ? embedding + (size_t)token_ids[r] * H : nullptr;
    const float* rrow = resid + (size_t)r * H;
    const bool one_batch = n4 <= kNormBatch * 32;
    float x[kNormBatch][4], w[kNormBatch][4];
    float ss = 0.f;
    if (one_batch) {                                       // the norm weight travels with the row, not after the sum
#pragma unroll
      for (int j = 0; j < kNormBatch; ++j)
        if (j * 32 + lane < n4) load4<float>(ln_w + (j * 32 + lane) * 4, w[j]);
    }
    for (int g0 = 0; g0 < n4; g0 += kNormBatch * 32) {
#pragma unroll
      for (int j = 0; j < kNormBatch; ++j) {
        const int g = g0 + j * 32 + lane;
        if (g < n4) fu_load_x4(erow, rrow, g * 4, x[j]);
        else x[j][0] = x[j][1] = x[j][2] = x[j][3] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < kNormBatch; ++j) ss += x[j][0] * x[j][0] + x[j][1] * x[j][1] + x[j][2] * x[j][2] + x[j][3] * x[j][3];
    }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    const bool writer = erow && (int)blockIdx.x == r % (int)gridDim.x;
    for (int g0 = 0; g0 < n4; g0 += kNormBatch * 32) {
      if (!one_batch) {                                    // wide rows: read the batch again
#pragma unroll
        for (int j = 0; j < kNormBatch; ++j) {
          const int g = g0 + j * 32 + lane;
          if (g < n4) fu_load_x4(erow, rrow, g * 4, x[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < kNormBatch; ++j) {
        const int g = g0 + j * 32 + lane;
        if (g >= n4) continue;
        if (writer) *reinterpret_cast<float4*>(resid + (size_t)r * H + g * 4) = make_float4(x[j][0], x[j][1], x[j][2], x[j][3]);
        float y[4];
        if (!one_batch) load4<float>(ln_w + g * 4, w[j]);
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = w[j][e] * __bfloat162float(__float2bfloat16_rn(x[j][e] * rstd));
        store4<__nv_bfloat16>(dst + g * 4, y);
      }
    }
  }
}

// ---- The projections ---------------------------------------------------------------------------------------
// The weight-streaming product of gemm_skinny_bf16.cu, shared out over the resident grid. A UNIT is 8 weight
// rows and, where the epilogue needs two rows per output (a rotation pair of q/k/v; a gate row and its up
// row), their 8 partner rows. The units are taken in passes; in a pass every block holds `upc` units (4, 2 or
// 1: as many as keep all blocks busy) and cuts K across the kw = 8 / upc warps of a unit; partial sums meet in
// shared memory in warp order, so the result does not depend on timing. A lane keeps kFuSlots pairs of
// 16-byte weight loads in flight. The first pass's first loads can be issued before a grid barrier is
// waited for (weights do not depend on other blocks), and an input other blocks wrote is staged by each
// warp for its own K range, so that neither costs a round trip of its own.
constexpr int kFuSlots = 7;

struct FuTask {
  int base, upc, kw;        // the pass: first unit, units per block, warps per unit
  int u;                    // this warp's unit (may be beyond n_units: then the warp loads nothing)
  int kpart, c_begin, c_end;
  const __nv_bfloat16* wa;  // the lane's row of the unit, and of the partner rows (or the same row)
  const __nv_bfloat16* wb;
  bool ok_a, ok_b;
};

template <int MODE>
__device__ __forceinline__ FuTask fu_task(const FusedArgs& a, const __nv_bfloat16* W, int N, int K, int n_units,
                                          int base) {
  constexpr bool PAIR = MODE != FU_ADD_RESID;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  FuTask t;
  t.base = base;
  const int per_block = (n_units - base) / (int)gridDim.x;
  t.upc = per_block >= 4 ? 4 : per_block >= 2 ? 2 : 1;
  t.kw = kFuWarps / t.upc;
  const int j = warp / t.kw;
  t.kpart = warp - j * t.kw;
  t.u = base + j * (int)gridDim.x + (int)blockIdx.x;
  const int n_chunks = (K + 31) / 32;
  const int per = (n_chunks + t.kw - 1) / t.kw;
  t.c_begin = t.kpart * per;
  t.c_end = min(n_chunks, t.c_begin + per);
  int row_a, row_b;
  if (MODE == FU_QKV) {
    const int per_head = a.D / 16;
    const int head = t.u / per_head;
    row_a = head * a.D + (t.u - head * per_head) * 8;
    row_b = row_a + a.D / 2;
  } else if (MODE == FU_SWIGLU) {
    row_a = t.u * 8;
    row_b = a.I + t.u * 8;
  } else {
    row_a = row_b = t.u * 8;
  }
  t.ok_a = t.ok_b = t.u < n_units;
  t.wa = fu_packed(W, t.ok_a ? row_a : 0, n_chunks, lane);
  t.wb = fu_packed(W, t.ok_b ? row_b : 0, n_chunks, lane);
  (void)PAIR;
  (void)N;
  return t;
}

// Slot s of a task: the two 16-byte loads that travel together. With partner rows they are the same K chunk of
// both rows; without, two neighbouring chunks of the one row.
template <int MODE>
__device__ __forceinline__ void fu_slot_chunks(const FuTask& t, int s, int& ca, int& cb) {
  if (MODE != FU_ADD_RESID) {
    ca = cb = t.c_begin + s;
  } else {
    ca = t.c_begin + 2 * s;
    cb = ca + 1;
  }
}

template <int MODE>
__device__ __forceinline__ void fu_slot_load(const FuTask& t, int K, int s, uint4& ra, uint4& rb) {
  int ca, cb;
  fu_slot_chunks<MODE>(t, s, ca, cb);
  (void)K;
  ra = (t.ok_a && ca < t.c_end) ? fu_ldg_stream(t.wa + (size_t)ca * kFuChunkElems) : make_uint4(0u, 0u, 0u, 0u);
  rb = (t.ok_b && cb < t.c_end) ? fu_ldg_stream(t.wb + (size_t)cb * kFuChunkElems) : make_uint4(0u, 0u, 0u, 0u);
}

// The first loads of a projection's first pass; call it between a barrier's arrival and its wait.
template <int MODE>
__device__ __forceinline__ void fu_project_preload(const FusedArgs& a, const __nv_bfloat16* W, int N, int K,
                                                   int n_units, uint4 (&ra)[kFuSlots], uint4 (&rb)[kFuSlots]) {
  const FuTask t = fu_task<MODE>(a, W, N, K, n_units, 0);
#pragma unroll
  for (int i = 0; i < kFuSlots; ++i) fu_slot_load<MODE>(t, K, i, ra[i], rb[i]);
}

// `stage_src`: null when the block's shared memory already holds the input (the norm wrote it), else the
// [T, K] bfloat16 matrix other blocks wrote (rows beyond T stay as they are: they only feed accumulator rows
// nobody reads). `preloaded`: ra / rb hold the first pass's first loads.
template <int MODE>
__device__ __forceinline__ void fu_project(const FusedArgs& a, const FusedLayer& L, const __nv_bfloat16* W, int N,
                                           int K, int n_units, const __nv_bfloat16* stage_src, unsigned char* xs,
                                           int row_bytes, float* red, bool preloaded, uint4 (&ra)[kFuSlots],
                                           uint4 (&rb)[kFuSlots]) {
  constexpr bool PAIR = MODE != FU_ADD_RESID;
  constexpr int U = kFuSlots;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned char* xrow = xs + (lane >> 2) * row_bytes + (lane & 3) * 16;
  // With at most 8 tokens only 8 rows are staged; the fragment rows 8..15 then read rows 0..7 again and
  // feed accumulator rows nobody reads.
  const size_t hi_off = a.T > 8 ? (size_t)8 * row_bytes : 0;
  for (int base = 0; base < n_units;) {
    const FuTask t = fu_task<MODE>(a, W, N, K, n_units, base);
    if (!(preloaded && base == 0)) {
#pragma unroll
      for (int i = 0; i < U; ++i) fu_slot_load<MODE>(t, K, i, ra[i], rb[i]);
    }
    if (stage_src && base == 0) {
      // Warp w brings in the K range that is its own when 8 warps share a unit.
      const int n_chunks = (K + 31) / 32;
      const int per8 = (n_chunks + kFuWarps - 1) / kFuWarps;
      const int c0 = warp * per8, c1 = min(n_chunks, c0 + per8);
      const uint32_t sbase = smem_u32(xs);
      const int pieces = max(0, c1 - c0) * 4;
      for (int idx = lane; idx < a.T * pieces; idx += 32) {
        const int r = idx / pieces, pc = idx - r * pieces;
        const int k = c0 * 32 + pc * 8;
        const bool ok = k < K;
        cp_async16(sbase + r * row_bytes + k * 2, ok ? stage_src + (size_t)r * K + k : stage_src, ok);
      }
      cp_async_commit();
    }
    // The residual element this thread will add to, asked for before the products (one owner per element).
    float resid_in = 0.f;
    if (!PAIR && tid < t.upc * a.T * 8) {
      const int j = tid / (a.T * 8), rem = tid - j * (a.T * 8);
      const int n = (base + j * (int)gridDim.x + (int)blockIdx.x) * 8 + (rem & 7);
      if (n < N) resid_in = __ldcg(a.resid + (size_t)(rem >> 3) * N + n);
    }
    float acc_a[4] = {0.f, 0.f, 0.f, 0.f}, acc_b[4] = {0.f, 0.f, 0.f, 0.f};
    const int n_slots = PAIR ? t.c_end - t.c_begin : (t.c_end - t.c_begin + 1) / 2;
    for (int s0 = 0; s0 < n_slots || s0 == 0; s0 += U) {
      uint4 ca[U], cb[U];
#pragma unroll
      for (int i = 0; i < U; ++i) {
        ca[i] = ra[i];
        cb[i] = rb[i];
      }
      if (s0 + U < n_slots) {
#pragma unroll
        for (int i = 0; i < U; ++i) fu_slot_load<MODE>(t, K, s0 + U + i, ra[i], rb[i]);
      }
      if (stage_src && base == 0 && s0 == 0) {             // the staged input is needed only now
        cp_async_wait<0>();
        if (t.kw == kFuWarps) __syncwarp(); else __syncthreads();   // uniform over the block
      }
#pragma unroll
      for (int i = 0; i < U; ++i) {
        if (s0 + i < n_slots) {
          int xa, xb;
          fu_slot_chunks<MODE>(t, s0 + i, xa, xb);
          const uint4 lo = *reinterpret_cast<const uint4*>(xrow + xa * 64);
          const uint4 hi = *reinterpret_cast<const uint4*>(xrow + hi_off + xa * 64);
          fu_mma(acc_a, lo.x, hi.x, lo.y, hi.y, ca[i].x, ca[i].y);
          fu_mma(acc_a, lo.z, hi.z, lo.w, hi.w, ca[i].z, ca[i].w);
          if (PAIR) {
            fu_mma(acc_b, lo.x, hi.x, lo.y, hi.y, cb[i].x, cb[i].y);
            fu_mma(acc_b, lo.z, hi.z, lo.w, hi.w, cb[i].z, cb[i].w);
          } else if (xb < t.c_end) {                       // uniform over the warp
            const uint4 lo2 = *reinterpret_cast<const uint4*>(xrow + xb * 64);
            const uint4 hi2 = *reinterpret_cast<const uint4*>(xrow + hi_off + xb * 64);
            fu_mma(acc_a, lo2.x, hi2.x, lo2.y, hi2.y, cb[i].x, cb[i].y);
            fu_mma(acc_a, lo2.z, hi2.z, lo2.w, hi2.w, cb[i].z, cb[i].w);
          }
        }
      }
    }
    // Partial sums: red[warp][row group][token][feature].
    {
      const int t0 = lane >> 2, f = (lane & 3) * 2;
      float* mine = red + (size_t)warp * 2 * 16 * 8;
      *reinterpret_cast<float2*>(mine + t0 * 8 + f) = make_float2(acc_a[0], acc_a[1]);
      *reinterpret_cast<float2*>(mine + (t0 + 8) * 8 + f) = make_float2(acc_a[2], acc_a[3]);
      if (PAIR) {
        *reinterpret_cast<float2*>(mine + 128 + t0 * 8 + f) = make_float2(acc_b[0], acc_b[1]);
        *reinterpret_cast<float2*>(mine + 128 + (t0 + 8) * 8 + f) = make_float2(acc_b[2], acc_b[3]);
      }
    }
    __syncthreads();
    const int kw = t.kw;
    auto total = [&](int j, int grp, int tok, int f) -> float {
      float sum = 0.f;
      for (int p = 0; p < kw; ++p) sum += red[(((size_t)(j * kw + p) * 2 + grp) * 16 + tok) * 8 + f];
      return sum;
    };
    for (int idx = tid; idx < t.upc * a.T * 8; idx += kFuThreads) {
      const int j = idx / (a.T * 8), rem = idx - j * (a.T * 8);
      const int tok = rem >> 3, f = rem & 7;
      const int u = base + j * (int)gridDim.x + (int)blockIdx.x;
      if (u >= n_units) continue;
      {
        // residual + branch, in 32-bit; each element has one owner, so the update is in place
        const int n = u * 8 + f;
        if (n < N) a.resid[(size_t)tok * N + n] = (idx == tid ? resid_in : __ldcg(a.resid + (size_t)tok * N + n)) + total(j, 0, tok, f);
      }
    }
    __syncthreads();   // `red` is reused by the next pass
    base += t.upc * (int)gridDim.x;
  }
}

// The QKV projection: a unit is 8 rows of one head and their 8 rotation partners (half a head further); a
// block takes one unit at a time, 4 warps per row group cutting K between them; bias, rotation and the
// writes of q and of the cache slots follow on the summed partials.
__device__ __forceinline__ void fu_qkv_units(const FusedArgs& a, const FusedLayer& L, const __nv_bfloat16* W, int N,
                                             int K, int n_units, const unsigned char* xs, int row_bytes, float* red) {
  constexpr int ng = 2;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kw = kFuWarps / ng;
  const int g = warp / kw, kpart = warp - g * kw;
  const int n_chunks = (K + 31) / 32;
  const int per = (n_chunks + kw - 1) / kw;
  const int c_begin = kpart * per, c_end = min(n_chunks, c_begin + per);
  const unsigned char* xrow = xs + (lane >> 2) * row_bytes + (lane & 3) * 16;
  // With at most 8 tokens only 8 rows are staged; the fragment rows 8..15 then read rows 0..7 again and
  // feed accumulator rows nobody reads.
  const size_t hi_off = a.T > 8 ? (size_t)8 * row_bytes : 0;
  constexpr int U = 8;
  for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
    const int per_head = a.D / 16;
    const int row0 = (u / per_head) * a.D + (u % per_head) * 8 + g * (a.D / 2);
    const __nv_bfloat16* wp = fu_packed(W, row0, n_chunks, lane);
    auto load_w = [&](int c) -> uint4 {
      if (c < c_end) return fu_ldg_stream(wp + (size_t)c * kFuChunkElems);
      return make_uint4(0u, 0u, 0u, 0u);
    };
    uint4 wreg[U];
#pragma unroll
    for (int i = 0; i < U; ++i) wreg[i] = load_w(c_begin + i);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = c_begin; c < c_end; c += U) {
      uint4 cur[U];
#pragma unroll
      for (int i = 0; i < U; ++i) cur[i] = wreg[i];
#pragma unroll
      for (int i = 0; i < U; ++i) wreg[i] = load_w(c + U + i);
#pragma unroll
      for (int i = 0; i < U; ++i) {
        if (c + i < c_end) {
          const uint4 lo = *reinterpret_cast<const uint4*>(xrow + (c + i) * 64);
          const uint4 hi = *reinterpret_cast<const uint4*>(xrow + hi_off + (c + i) * 64);
          fu_mma(acc, lo.x, hi.x, lo.y, hi.y, cur[i].x, cur[i].y);
          fu_mma(acc, lo.z, hi.z, lo.w, hi.w, cur[i].z, cur[i].w);
        }
      }
    }
    {
      const int t0 = lane >> 2, f = (lane & 3) * 2;
      *reinterpret_cast<float2*>(red + ((size_t)warp * 16 + t0) * 8 + f) = make_float2(acc[0], acc[1]);
      *reinterpret_cast<float2*>(red + ((size_t)warp * 16 + t0 + 8) * 8 + f) = make_float2(acc[2], acc[3]);
    }
    __syncthreads();
    auto total = [&](int t, int grp, int f) -> float {
      float s = 0.f;
      for (int p = 0; p < kw; ++p) s += red[((size_t)(grp * kw + p) * 16 + t) * 8 + f];
      return s;
    };
    {
      const int half = a.D / 2;
      const int head = u / per_head, i0 = (u - head * per_head) * 8;
      for (int idx = tid; idx < a.T * 8; idx += kFuThreads) {
        const int t = idx >> 3, j = idx & 7, i = i0 + j;
        const int c0 = head * a.D + i, c1 = c0 + half;
        float x1 = total(t, 0, j), x2 = total(t, 1, j);
        if (L.b_qkv) {
          x1 += L.b_qkv[c0];
          x2 += L.b_qkv[c1];
        }
        float o1 = x1, o2 = x2;
        if (head < a.nh + a.nkv) {
          int pos = a.positions[t];
          pos = pos < 0 ? 0 : (pos >= a.n_pos ? a.n_pos - 1 : pos);
          const float cs = a.cos_t[(size_t)pos * half + i], sn = a.sin_t[(size_t)pos * half + i];
          o1 = __fadd_rn(__fmul_rn(x1, cs), __fmul_rn(-x2, sn));
          o2 = __fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn));
        }
        if (head < a.nh) {
          __nv_bfloat16* dst = a.q + ((size_t)t * a.nh + head) * a.D;
          dst[i] = __float2bfloat16_rn(o1);
          dst[i + half] = __float2bfloat16_rn(o2);
        } else {
          const int slot = a.slot_map[t];
          if (slot >= 0) {
            const bool is_k = head < a.nh + a.nkv;
            const int kh = is_k ? head - a.nh : head - a.nh - a.nkv;
            __nv_bfloat16* dst = (is_k ? L.kcache : L.vcache) + ((size_t)slot * a.nkv + kh) * a.D;
            dst[i] = __float2bfloat16_rn(o1);
            dst[i + half] = __float2bfloat16_rn(o2);
          }
        }
      }
    }
    __syncthreads();   // `red` is reused by the next unit
  }
}

// The gate/up projection with SwiGLU: one WARP owns a unit of 8 gate rows and their 8 up rows over the whole K
// range, so there is no partial sum to meet in shared memory and no block-wide synchronisation; the
// activation is computed on the accumulator registers. (Streaming is bound by the loads a block keeps in
// flight; cutting K across warps to use the idle ones was tried and lost more to the extra pass and its
// synchronisation than it gained.)
__device__ __forceinline__ void fu_gate_up_units(const FusedArgs& a, const __nv_bfloat16* W, int N, int K, int n_units,
                                                 const unsigned char* xs, int row_bytes) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t2 = (lane & 3) * 2;
  const int n_chunks = (K + 31) / 32;
  const unsigned char* xrow = xs + g * row_bytes + (lane & 3) * 16;
  // With at most 8 tokens only 8 rows are staged; the fragment rows 8..15 then read rows 0..7 again and
  // feed accumulator rows nobody reads.
  const size_t hi_off = a.T > 8 ? (size_t)8 * row_bytes : 0;
  constexpr int U = 6;
  // Unit u goes to warp (u / grid) of block (u % grid): consecutive units land on different SMs.
  for (int u = warp * gridDim.x + blockIdx.x; u < n_units; u += kFuWarps * gridDim.x) {
    const int row_a = u * 8, row_b = a.I + u * 8;
    const bool ok_a = true, ok_b = true;
    const __nv_bfloat16* wa = fu_packed(W, row_a, n_chunks, lane);
    const __nv_bfloat16* wb = fu_packed(W, row_b, n_chunks, lane);
    auto load = [&](const __nv_bfloat16* p, bool ok, int c) -> uint4 {
      if (ok && c < n_chunks) return fu_ldg_stream(p + (size_t)c * kFuChunkElems);
      return make_uint4(0u, 0u, 0u, 0u);
    };
    uint4 ra[U], rb[U];
#pragma unroll
    for (int i = 0; i < U; ++i) {
      ra[i] = load(wa, ok_a, i);
      rb[i] = load(wb, ok_b, i);
    }
    float acc_a[4] = {0.f, 0.f, 0.f, 0.f}, acc_b[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = 0; c < n_chunks; c += U) {
      uint4 ca[U], cb[U];
#pragma unroll
      for (int i = 0; i < U; ++i) {
        ca[i] = ra[i];
        cb[i] = rb[i];
      }
#pragma unroll
      for (int i = 0; i < U; ++i) {
        ra[i] = load(wa, ok_a, c + U + i);
        rb[i] = load(wb, ok_b, c + U + i);
      }
#pragma unroll
      for (int i = 0; i < U; ++i) {
        if (c + i < n_chunks) {
          const uint4 lo = *reinterpret_cast<const uint4*>(xrow + (c + i) * 64);
          const uint4 hi = *reinterpret_cast<const uint4*>(xrow + hi_off + (c + i) * 64);
          fu_mma(acc_a, lo.x, hi.x, lo.y, hi.y, ca[i].x, ca[i].y);
          fu_mma(acc_a, lo.z, hi.z, lo.w, hi.w, ca[i].z, ca[i].w);
          fu_mma(acc_b, lo.x, hi.x, lo.y, hi.y, cb[i].x, cb[i].y);
          fu_mma(acc_b, lo.z, hi.z, lo.w, hi.w, cb[i].z, cb[i].w);
        }
      }
    }
    // Accumulator layout: [0], [1] = token g, features t2, t2 + 1; [2], [3] = token g + 8, same features.
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int t = g + hh * 8;
      if (t >= a.T) continue;
      float v1[2] = {acc_a[2 * hh], acc_a[2 * hh + 1]}, v2[2] = {acc_b[2 * hh], acc_b[2 * hh + 1]};
      {
        const int n = u * 8 + t2;
        if (n + 1 < a.I) {
          *reinterpret_cast<uint32_t*>(a.act + (size_t)t * a.I + n) =
              pack_bf16(v1[0] / (1.0f + expf(-v1[0])) * v2[0], v1[1] / (1.0f + expf(-v1[1])) * v2[1]);
        } else if (n < a.I) {
          a.act[(size_t)t * a.I + n] = __float2bfloat16_rn(v1[0] / (1.0f + expf(-v1[0])) * v2[0]);
        }
      }
    }
  }
}

// ---- Attention --------------------------------------------------------------------------------------------
// A unit is (request, kv head, key split) and belongs to one block. Its keys are shared out evenly over the 8
// warps; a warp brings its own keys and values into its own slice of shared memory (all of them in flight at
// once, up to kFuKeyCap or what the slice holds, in rounds beyond that) and works through them 16 keys at a
// time with the online softmax of attention_decode_bf16.cu, with nothing to wait for but its own copies.
// The 8 warps' states then meet in shared memory in warp order. With one split per request (the usual case:
// the host splits only long contexts) the block writes the head outputs itself; with more, it writes a
// partial and the block that finishes a (request, kv head) last merges the partials in split order.
constexpr int kFuKeyCap = 96;      // keys per warp whose cache slots are looked up once per launch

struct FuAttnUnit {
  int s, kvh, z, q_start, q_len, before, n_rows;
  int j_lo, j_hi;               // the unit's key range (inclusive); empty when j_lo > j_hi
  int kpw;                      // keys per warp (a multiple of 16)
};

__device__ __forceinline__ FuAttnUnit fu_attn_unit(const FusedArgs& a, int u, const int* s_cu_q, const int* s_before) {
  FuAttnUnit t;
  t.z = u % a.max_splits;
  const int sk = u / a.max_splits;
  t.kvh = sk % a.nkv;
  t.s = sk / a.nkv;
  t.q_start = s_cu_q[t.s];
  t.q_len = s_cu_q[t.s + 1] - t.q_start;
  t.before = s_before[t.s];
  const int G = a.nh / a.nkv;
  t.n_rows = min(t.q_len * G, 16);
  const int p_min = t.before, p_max = t.before + (t.n_rows - 1) / G;
  int lo = a.window > 0 ? max(0, p_min - a.window + 1) : 0;
  t.j_lo = max(lo, t.z * a.split_keys);
  t.j_hi = t.n_rows > 0 ? min(p_max, (t.z + 1) * a.split_keys - 1) : -1;
  const int n = t.j_hi - t.j_lo + 1;
  t.kpw = n > 0 ? ((n + kFuWarps - 1) / kFuWarps + 15) / 16 * 16 : 16;
  return t;
}

__device__ __forceinline__ int fu_slot_of(const FusedArgs& a, int s, int j) {
  const int page = a.block_table[(size_t)s * a.bt_stride + j / a.page_size];
  return page < 0 ? -1 : page * a.page_size + j % a.page_size;
}

template <int D>
__device__ __forceinline__ void fu_attention(const FusedArgs& a, const FusedLayer& L, unsigned char* smem,
                                             int smem_bytes, const int* s_cu_q, const int* s_before,
                                             const int (*s_slot)[kFuKeyCap], int layer) {
  constexpr int CH = D / 8, KS = D / 16, NT = D / 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = a.nh / a.nkv;
  const int r0 = lane >> 2, r1 = r0 + 8, cpair = (lane & 3) * 2;
  // Keys a warp's slice of shared memory holds (K rows then V rows), a multiple of 16.
  const int cap = (smem_bytes / kFuWarps) / (2 * D * 2) / 16 * 16;
  const uint32_t k_base = smem_u32(smem) + warp * (cap * 2 * D * 2), v_base = k_base + cap * D * 2;
  __shared__ int s_last;
  const int n_units = a.S * a.nkv * a.max_splits;
  for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
    const FuAttnUnit t = fu_attn_unit(a, u, s_cu_q, s_before);
    if (t.j_lo > t.j_hi) continue;                       // uniform over the block
    const int w_lo = t.j_lo + warp * t.kpw, w_hi = min(t.j_hi, w_lo + t.kpw - 1);
    const bool cached = u == (int)blockIdx.x;            // the launch-time slot table covers the first unit

    uint32_t qa[KS][4];
    {
      const __nv_bfloat16* qr0 = nullptr;
      const __nv_bfloat16* qr1 = nullptr;
      if (r0 < t.n_rows) qr0 = a.q + ((size_t)(t.q_start + r0 / G) * a.nh + t.kvh * G + r0 % G) * D;
      if (r1 < t.n_rows) qr1 = a.q + ((size_t)(t.q_start + r1 / G) * a.nh + t.kvh * G + r1 % G) * D;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const int c = ks * 16 + cpair;
        qa[ks][0] = qr0 ? __ldcg(reinterpret_cast<const unsigned int*>(qr0 + c)) : 0u;
        qa[ks][1] = qr1 ? __ldcg(reinterpret_cast<const unsigned int*>(qr1 + c)) : 0u;
        qa[ks][2] = qr0 ? __ldcg(reinterpret_cast<const unsigned int*>(qr0 + c + 8)) : 0u;
        qa[ks][3] = qr1 ? __ldcg(reinterpret_cast<const unsigned int*>(qr1 + c + 8)) : 0u;
      }
    }
    const int p_r0 = r0 < t.n_rows ? t.before + r0 / G : -1, p_r1 = r1 < t.n_rows ? t.before + r1 / G : -1;
    const int lo_r0 = a.window > 0 ? max(0, p_r0 - a.window + 1) : 0;
    const int lo_r1 = a.window > 0 ? max(0, p_r1 - a.window + 1) : 0;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // running max (log2 units) and sum per row
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    for (int kb = w_lo; kb <= w_hi; kb += cap) {         // rounds: usually one
      const int nk = min(cap, w_hi - kb + 1);
      const int nk16 = (nk + 15) / 16 * 16;
      for (int idx = lane; idx < nk16 * CH; idx += 32) {
        const int row = idx / CH, c = idx - row * CH;
        int slot = -1;
        if (row < nk) slot = (cached && kb == w_lo && row < kFuKeyCap) ? s_slot[warp][row] : fu_slot_of(a, t.s, kb + row);
        const bool ok = slot >= 0;
        const size_t src = ok ? ((size_t)slot * a.nkv + t.kvh) * D + c * 8 : 0;
        const uint32_t off = row * (D * 2) + ((c ^ (row & 7)) << 4);
        cp_async16(k_base + off, L.kcache + src, ok);      // rows without a key are filled with zeros
        cp_async16(v_base + off, L.vcache + src, ok);
      }
      cp_async_commit();
      if (u == (int)blockIdx.x) fu_stamp(a, layer * 16 + 10);
      cp_async_wait<0>();
      __syncwarp();
      if (u == (int)blockIdx.x) fu_stamp(a, layer * 16 + 11);
      for (int kr = 0; kr < nk; kr += 16) {
        float sc[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
        {
          const int key = kr + (lane & 7) + ((lane >> 4) << 3);
          const int csel = (lane >> 3) & 1;
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(k_base + key * (D * 2) + (((2 * ks + csel) ^ (key & 7)) << 4), b0, b1, b2, b3);
            mma_bf16_16816(sc[0], qa[ks], b0, b1);
            mma_bf16_16816(sc[1], qa[ks], b2, b3);
          }
        }
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = kb + kr + i * 8 + cpair + e;
            const bool in = j <= w_hi;
            sc[i][e] = (in && j <= p_r0 && j >= lo_r0) ? sc[i][e] * a.scale_log2 : -INFINITY;
            sc[i][2 + e] = (in && j <= p_r1 && j >= lo_r1) ? sc[i][2 + e] * a.scale_log2 : -INFINITY;
            tmax0 = fmaxf(tmax0, sc[i][e]);
            tmax1 = fmaxf(tmax1, sc[i][2 + e]);
          }
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
        const float mn0 = fmaxf(m0, tmax0), mn1 = fmaxf(m1, tmax1);
        const float corr0 = mn0 == -INFINITY ? 1.f : exp2f(m0 - mn0), corr1 = mn1 == -INFINITY ? 1.f : exp2f(m1 - mn1);
        float ps0 = 0.f, ps1 = 0.f;
        uint32_t pa[4];
        {
          float p[2][4];
#pragma unroll
          for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              p[i][e] = mn0 == -INFINITY ? 0.f : exp2f(sc[i][e] - mn0);
              p[i][2 + e] = mn1 == -INFINITY ? 0.f : exp2f(sc[i][2 + e] - mn1);
              ps0 += p[i][e];
              ps1 += p[i][2 + e];
            }
          pa[0] = pack_bf16(p[0][0], p[0][1]);
          pa[1] = pack_bf16(p[0][2], p[0][3]);
          pa[2] = pack_bf16(p[1][0], p[1][1]);
          pa[3] = pack_bf16(p[1][2], p[1][3]);
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
        for (int i = 0; i < NT; ++i) {
          o[i][0] *= corr0;
          o[i][1] *= corr0;
          o[i][2] *= corr1;
          o[i][3] *= corr1;
        }
        {
          const int key = kr + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int csel = lane >> 4;
#pragma unroll
          for (int dt = 0; dt < NT / 2; ++dt) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(v_base + key * (D * 2) + (((2 * dt + csel) ^ (key & 7)) << 4), b0, b1, b2, b3);
            mma_bf16_16816(o[2 * dt], pa, b0, b1);
            mma_bf16_16816(o[2 * dt + 1], pa, b2, b3);
          }
        }
      }
      __syncwarp();                                        // the slice is refilled by the next round
    }

    // The 8 warps' states meet in warp order: [warp][16 rows][D] sums, then [warp][16][2] (max, sum).
    if (u == (int)blockIdx.x) fu_stamp(a, layer * 16 + 12);
    __syncthreads();
    if (u == (int)blockIdx.x) fu_stamp(a, layer * 16 + 13);
    float* macc = reinterpret_cast<float*>(smem);
    float* mml = macc + kFuWarps * 16 * D;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int c = i * 8 + cpair;
      *reinterpret_cast<float2*>(macc + (warp * 16 + r0) * D + c) = make_float2(o[i][0], o[i][1]);
      *reinterpret_cast<float2*>(macc + (warp * 16 + r1) * D + c) = make_float2(o[i][2], o[i][3]);
    }
    if ((lane & 3) == 0) {
      mml[(warp * 16 + r0) * 2] = m0;
      mml[(warp * 16 + r0) * 2 + 1] = l0;
      mml[(warp * 16 + r1) * 2] = m1;
      mml[(warp * 16 + r1) * 2 + 1] = l1;
    }
    __syncthreads();
    constexpr float kLn2 = 0.6931471805599453f;
    for (int idx = tid; idx < t.n_rows * (D / 2); idx += kFuThreads) {
      const int r = idx / (D / 2), d = (idx - r * (D / 2)) * 2;
      float mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < kFuWarps; ++w) mx = fmaxf(mx, mml[(w * 16 + r) * 2]);
      float acc0 = 0.f, acc1 = 0.f, lsum = 0.f;
#pragma unroll
      for (int w = 0; w < kFuWarps; ++w) {
        const float mw = mml[(w * 16 + r) * 2];
        const float wgt = mw == -INFINITY ? 0.f : exp2f(mw - mx);
        const float2 v = *reinterpret_cast<const float2*>(macc + (w * 16 + r) * D + d);
        acc0 = fmaf(v.x, wgt, acc0);
        acc1 = fmaf(v.y, wgt, acc1);
        lsum = fmaf(mml[(w * 16 + r) * 2 + 1], wgt, lsum);
      }
      const size_t orow = (size_t)(t.q_start + r / G) * a.nh + t.kvh * G + r % G;
      if (a.max_splits == 1) {
        *reinterpret_cast<uint32_t*>(a.attn + orow * D + d) = pack_bf16(acc0 / lsum, acc1 / lsum);
      } else {
        *reinterpret_cast<float2*>(a.part_acc + (orow * a.max_splits + t.z) * D + d) = make_float2(acc0, acc1);
        if (d == 0) {
          a.part_ml[(orow * a.max_splits + t.z) * 2] = mx * kLn2;     // natural-log units
          a.part_ml[(orow * a.max_splits + t.z) * 2 + 1] = lsum;
        }
      }
    }
    if (u == (int)blockIdx.x) fu_stamp(a, layer * 16 + 14);
    if (a.max_splits > 1) {
      // How many splits hold keys for this (request, kv head): the last one to finish merges them.
      const int p_max = t.before + (t.n_rows - 1) / G;
      const int lo_all = a.window > 0 ? max(0, t.before - a.window + 1) : 0;
      const int expected = p_max / a.split_keys - lo_all / a.split_keys + 1;
      __threadfence();
      __syncthreads();
      if (tid == 0) s_last = atomicAdd(&a.attn_count[t.s * a.nkv + t.kvh], 1) == expected - 1;
      __syncthreads();
      if (s_last) {
        __threadfence();
        for (int idx = tid; idx < t.n_rows * (D / 4); idx += kFuThreads) {
          const int r = idx / (D / 4), d = (idx - r * (D / 4)) * 4;
          const size_t orow = (size_t)(t.q_start + r / G) * a.nh + t.kvh * G + r % G;
          const int p = t.before + r / G;
          const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
          const int z0 = lo / a.split_keys, z1 = p / a.split_keys;
          // One pass in split order: the running maximum rescales what has been summed so far. The loads do
          // not depend on the running state, so several splits are in flight at a time.
          float mx = -INFINITY, lsum = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
          for (int zz = z0; zz <= z1; ++zz) {
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(a.part_ml + (orow * a.max_splits + zz) * 2));
            const float4 pa = __ldcg(reinterpret_cast<const float4*>(a.part_acc + (orow * a.max_splits + zz) * D + d));
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
          const float inv = 1.0f / lsum;
          uint2 ov;
          ov.x = pack_bf16(acc[0] * inv, acc[1] * inv);
          ov.y = pack_bf16(acc[2] * inv, acc[3] * inv);
          *reinterpret_cast<uint2*>(a.attn + orow * D + d) = ov;
        }
        if (tid == 0) a.attn_count[t.s * a.nkv + t.kvh] = 0;
      }
    }
    __syncthreads();   // s_last and the shared memory are reused by the next unit
  }
}

template <int D>
__global__ void __launch_bounds__(kFuThreads, 1) decode_fused_kernel(const FusedArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  const int kmax = max(a.H, max(a.nh * a.D, a.I));
  const int xs_bytes = (a.T > 8 ? 16 : 8) * fu_row_bytes(kmax);
  unsigned char* xs = smem;
  float* red = reinterpret_cast<float*>(smem + xs_bytes);            // [8 warps][2 row groups][16][8]
  const int rb_h = fu_row_bytes(a.H), rb_q = fu_row_bytes(a.nh * a.D), rb_i = fu_row_bytes(a.I);
  unsigned k = 0;
  bool ok = true;
  const int qkv_rows = (a.nh + 2 * a.nkv) * a.D;
  __syncthreads();

  auto packed_bytes = [](int n, int kk) { return (size_t)((n + 7) / 8 * 8) * ((kk + 31) / 32 * 32) * 2; };
  const size_t qkv_bytes = packed_bytes(qkv_rows, a.H), o_bytes = packed_bytes(a.H, a.nh * a.D);
  const size_t gu_bytes = packed_bytes(2 * a.I, a.H), down_bytes = packed_bytes(a.H, a.I);
  uint4 ra[kFuSlots], rb[kFuSlots];          // the projections' weight loads in flight
  __shared__ FusedLayer s_layer[2];          // this layer's pointers and the next one's, fetched a phase early
  if (threadIdx.x == 0 && a.n_layers > 0) s_layer[0] = a.layers[0];
  // The requests' lengths, and the cache slots of this block's first attention unit, are the same in every
  // layer: look them up once, so that each layer can ask for its keys and values a phase before it reads
  // them and starts its copies without a table lookup.
  __shared__ int s_cu_q[17], s_before[16];
  __shared__ int s_slot[kFuWarps][kFuKeyCap];
  if (threadIdx.x <= a.S) s_cu_q[threadIdx.x] = a.cu_q[threadIdx.x];
  if (threadIdx.x < a.S) s_before[threadIdx.x] = a.kv_before[threadIdx.x];
  __syncthreads();
  int first_kvh = 0;
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool live = (int)blockIdx.x < a.S * a.nkv * a.max_splits;
    FuAttnUnit t = {};
    if (live) t = fu_attn_unit(a, blockIdx.x, s_cu_q, s_before);
    first_kvh = t.kvh;
    const int w_lo = t.j_lo + warp * t.kpw, w_hi = min(t.j_hi, w_lo + t.kpw - 1);
    for (int i = lane; i < kFuKeyCap; i += 32)
      s_slot[warp][i] = (live && w_lo + i <= w_hi) ? fu_slot_of(a, t.s, w_lo + i) : -1;
  }
  __syncthreads();

  for (int l = 0; l < a.n_layers && ok; ++l) {
    const FusedLayer& L = s_layer[l & 1];
    fu_stamp(a, l * 16 + 0);
    fu_prefetch_l2(L.w_o, o_bytes);
    fu_prefetch_l2(L.w_gu, gu_bytes);
    for (int i = threadIdx.x & 31; i < kFuKeyCap; i += 32) {
      const int slot = s_slot[threadIdx.x >> 5][i];
      if (slot >= 0) {
        const size_t off = ((size_t)slot * a.nkv + first_kvh) * D;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(L.kcache + off));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(L.vcache + off));
        if (D > 64) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(L.kcache + off + 64));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(L.vcache + off + 64));
        }
      }
    }
    // A: norm + QKV
    fu_norm_rows(a.T, a.H, l == 0 ? a.embedding : nullptr, a.token_ids, a.resid, L.ln1_w, a.eps1, xs, rb_h);
    __syncthreads();
    fu_stamp(a, l * 16 + 1);
    fu_qkv_units(a, L, L.w_qkv, qkv_rows, a.H, (a.nh + 2 * a.nkv) * (a.D / 16), xs, rb_h, red);
    fu_stamp(a, l * 16 + 2);
    if (!(ok = fu_grid_sync(a, k, &s_ok))) break;
    fu_stamp(a, l * 16 + 3);
    // B: attention
    fu_attention<D>(a, L, smem, a.smem_bytes, s_cu_q, s_before, s_slot, l);
    fu_stamp(a, l * 16 + 4);
    // C: output projection; its first weights are asked for while the barrier fills up
    fu_grid_arrive(a);
    fu_project_preload<FU_ADD_RESID>(a, L.w_o, a.H, a.nh * a.D, (a.H + 7) / 8, ra, rb);
    fu_prefetch_l2(L.w_down, down_bytes);
    if (l + 1 < a.n_layers) {
      if (threadIdx.x == 0) s_layer[(l + 1) & 1] = a.layers[l + 1];
      fu_prefetch_l2(a.layers[l + 1].w_qkv, qkv_bytes);
    }
    if (!(ok = fu_grid_wait(a, k, &s_ok))) break;
    fu_stamp(a, l * 16 + 5);
    fu_project<FU_ADD_RESID>(a, L, L.w_o, a.H, a.nh * a.D, (a.H + 7) / 8, a.attn, xs, rb_q, red, true, ra, rb);
    fu_stamp(a, l * 16 + 6);
    if (!(ok = fu_grid_sync(a, k, &s_ok))) break;
    // D: norm + gate/up + SwiGLU
    fu_norm_rows(a.T, a.H, nullptr, a.token_ids, a.resid, L.ln2_w, a.eps2, xs, rb_h);
    __syncthreads();
    fu_stamp(a, l * 16 + 7);
    fu_gate_up_units(a, L.w_gu, 2 * a.I, a.H, (a.I + 7) / 8, xs, rb_h);
    fu_stamp(a, l * 16 + 8);
    // E: down projection, begun the same way
    fu_grid_arrive(a);
    fu_project_preload<FU_ADD_RESID>(a, L.w_down, a.H, a.I, (a.H + 7) / 8, ra, rb);
    if (!(ok = fu_grid_wait(a, k, &s_ok))) break;
    fu_project<FU_ADD_RESID>(a, L, L.w_down, a.H, a.I, (a.H + 7) / 8, a.act, xs, rb_i, red, true, ra, rb);
    fu_stamp(a, l * 16 + 9);
    if (!(ok = fu_grid_sync(a, k, &s_ok))) break;
  }
  fu_stamp(a, a.n_layers * 16);

  if (ok) {
    // Final norm of the wanted rows: block i takes wanted rows i, i + grid, ...; one warp per row.
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int w = blockIdx.x * kFuWarps + warp; w < a.n_want; w += gridDim.x * kFuWarps) {
      const int r = a.want_rows[w];
      const float* rrow = a.resid + (size_t)r * a.H;
      float ss = 0.f;
      for (int i = lane; i < a.H; i += 32) {
        const float x = __ldcg(rrow + i);
        ss += x * x;
      }
      ss = warp_sum(ss);
      const float rstd = 1.0f / sqrtf(ss / (float)a.H + a.eps_f);
      for (int i = lane; i < a.H; i += 32) {
        const float x = __ldcg(rrow + i);
        const __nv_bfloat16 normed = __float2bfloat16_rn(x * rstd);
        a.hidden_out[(size_t)w * a.H + i] = __float2bfloat16_rn(a.final_ln_w[i] * __bfloat162float(normed));
      }
    }
  }
  // Leave: the last block to get here puts the arrival counter back to zero (nobody waits on it any more).
  __syncthreads();
  if (threadIdx.x == 0 && ok) {
    __threadfence();
    const unsigned after = atomicAdd(a.bar, 1u) + 1;
    if (after == (k + 1) * gridDim.x) atomicExch(a.bar, 0u);
  }
}

template <int D>
int launch_decode_fused(const FusedArgs& a, cudaStream_t stream) {
  auto kern = decode_fused_kernel<D>;
  const int kmax = a.H > a.I ? (a.H > a.nh * a.D ? a.H : a.nh * a.D) : (a.I > a.nh * a.D ? a.I : a.nh * a.D);
  const int kpad = (kmax + 31) / 32 * 32;
  const int row_bytes = kpad * 2 + ((64 - (kpad * 2) % 128) + 128) % 128;
  // Less shared memory leaves more L1, and with it more loads in flight: steps of at most 8 tokens stage 8 rows.
  const int need = (a.T > 8 ? 16 : 8) * row_bytes + kFuWarps * 2 * 16 * 8 * (int)sizeof(float);
  // The attention warps use the same memory for keys in flight (at least 16 keys per warp) and then for
  // the 8 warps' states.
  constexpr int kAttnMin = kFuWarps * 16 * (D + 2) * 4 > kFuWarps * 16 * 4 * D ? kFuWarps * 16 * (D + 2) * 4 : kFuWarps * 16 * 4 * D;
  const int smem = need > kAttnMin ? need : kAttnMin;
  if (smem > 216 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
  static int n_sm = 0, per_sm = 0, smem_set = 0;
  if (smem > smem_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    smem_set = smem;
    per_sm = 0;
  }
  if (!per_sm) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kFuThreads, smem);
    if (e != cudaSuccess) return (int)e;
    if (per_sm < 1) return TM_ERR_UNSUPPORTED_SHAPE;
  }
  FusedArgs args = a;
  args.smem_bytes = smem;
  void* params[] = {&args};
  return (int)cudaLaunchCooperativeKernel((void*)kern, dim3(n_sm), dim3(kFuThreads), params, (size_t)smem, stream);
}

}  // namespace tmk

// `args` points to a host copy of tmk::FusedArgs (built by the caller field by field, see
// tokenmill_b200/kernels/fused.py). Conditions: bfloat16, T <= 16 tokens, every request at most 16 / (nh / nkv)
// tokens, head size 64 or 128, H, I and nh * D multiples of 8, one cache group.
extern "C" int tm_decode_fused(const void* args, cudaStream_t stream) {
  const tmk::FusedArgs& a = *reinterpret_cast<const tmk::FusedArgs*>(args);
  if (a.T <= 0) return 0;
  if (a.T > 16 || a.H % 8 || a.I % 8 || (a.nh * a.D) % 8 || a.nkv <= 0 || a.nh % a.nkv || a.nh / a.nkv > 16 ||
      a.split_keys <= 0 || a.max_splits <= 0 || a.S <= 0 || a.S > 16 || !a.bar || !a.error)
    return TM_ERR_UNSUPPORTED_SHAPE;
  if (a.D == 64) return tmk::launch_decode_fused<64>(a, stream);
  if (a.D == 128) return tmk::launch_decode_fused<128>(a, stream);
  return TM_ERR_UNSUPPORTED_SHAPE;
}

extern "C" int tm_decode_fused_args_size() { return (int)sizeof(tmk::FusedArgs); }
extern "C" int tm_decode_fused_layer_size() { return (int)sizeof(tmk::FusedLayer); }
