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
// Weights never wait for a phase: every block knows from the start which pieces of which matrices it will
// multiply, in which order, for the whole launch. It streams them through a ring of shared-memory stages with
// bulk asynchronous copies (cp.async.bulk, completion on an mbarrier per stage), a few stages ahead of the
// arithmetic and across phase and layer boundaries; the warps that used a stage up ask for the piece that
// comes next into it. Inputs that other blocks wrote (head outputs, activations) come in the same way, one
// bulk copy per token row, after the grid barrier that makes them complete. A measurement on this machine decided the form: a warp reading 8 rows x 64 bytes of a
// row-major matrix gets about 20 GB/s per SM out of L2, 512 contiguous bytes per warp load about 50 GB/s,
// bulk copies of 14 KB and more about 90 GB/s, bulk copies of a single 1.8 KB row 20 GB/s again. So the
// matrices are read from a packed copy (see fu_packed_group) in which the 8 rows a warp multiplies at a time
// are contiguous, in the order the tensor-core fragments want them.
//
// Phases per layer (the formulas are those of the separate kernels, which stay the reference for tests:
// norm.cu, gemm_skinny_bf16.cu, attention_decode_bf16.cu; reference model: src/infer/model/qwen2.py:13-23,
// src/infer/model/layers.py:127-164):
//   A  every block norms the residual stream (the embedding rows in the first layer) for all tokens into
//      shared memory; then the blocks share the QKV weight rows (8 rows and their 8 rotation partners per
//      unit, K cut across the 8 warps), add bias, rotate, and write q and the cache slots.
//   B  attention units (request, kv head, key split), one block each; the block that finishes a (request,
//      kv head) last merges the splits in index order and writes the head outputs.
//   C  output projection from the staged head outputs, added into the 32-bit residual stream.
//   D  as A with the second norm, then gate/up + SwiGLU (a warp per unit) into a [T, I] buffer.
//   E  down projection, added into the residual stream.
// Data written by other blocks is read with L2-level loads (ld.global.cg / cp.async.cg), since L1 is not
// coherent across SMs within a launch; weights are read-only.
//
// Every wait is bounded: a block that waits too long at the grid barrier or for a stage raises the error
// word, stops working and leaves; the others run into the same limit and leave too. Before leaving, a block
// waits (bounded again) for the copies it still has in flight. The launch is cooperative, so all blocks are
// resident together. The arrival counter is put back to zero by the last block to leave.
#include "mma_util.cuh"

namespace tmk {

constexpr int kFuThreads = 256;
constexpr int kFuWarps = 8;
constexpr uint32_t kFuSpinLimit = 1u << 22;
constexpr int kFuMaxStages = 8;
constexpr int kFuMaxLayers = 96;

struct FusedLayer {
  const float* ln1_w;
  // the four matrices in the packed layout described at fu_packed_group()
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
  const int* token_rows;           // null, or [T]: token t's id is token_ids[token_rows[t]] (ids left on the device by the previous step's sampling)
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
  int stage_bytes;                 // bytes of one stage of the weight ring (set by the launcher)
  int halves;                      // nonzero (set by the launcher): the down projection takes its 9..16 input rows 8 at a time
  unsigned long long* timing;      // null, or [n_layers * 16 + 1] nanosecond stamps written by block 0 (profiling aid)
};

__device__ __forceinline__ void fu_stamp(const FusedArgs& a, int slot) {
  if (a.timing && blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    a.timing[slot] = t;
  }
}

__device__ __forceinline__ void fu_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 fu_lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// The weights are read in a packed copy (made once, when the decoder is set up): for every group of 8 rows
// and every chunk of 32 columns, the 32 lanes' 16-byte pieces lie one after the other in lane order (lane
// 4 g + t holds row g, columns 8 t .. 8 t + 7 of the chunk; rows and columns beyond the matrix are zeros).
// A group's chunks follow one another, so any range of chunks of a group is one contiguous piece of
// 512 bytes per chunk: one bulk copy, and in shared memory a warp's fragment load is 512 contiguous bytes.
constexpr int kFuChunkElems = 32 * 8;
constexpr int kFuChunkBytes = 512;
__device__ __forceinline__ const __nv_bfloat16* fu_packed_group(const __nv_bfloat16* W, int row0, int n_chunks, int chunk) {
  return W + ((size_t)(row0 >> 3) * n_chunks + chunk) * kFuChunkElems;
}

// Where element d of a query row lies in the kernel's own q buffer: lane 4 g + t of the attention phase reads, for
// every 16-wide step ks of the head dimension, elements 16 ks + 2 t + {0, 1, 8, 9} of its rows; they are stored
// as t's block [ks][0, 1, 8, 9], so that a lane's fragments of a row are D / 4 contiguous elements.
__device__ __forceinline__ int fu_q_index(int d, int D) {
  const int ks = d >> 4, rem = d & 15;
  return ((rem & 7) >> 1) * (D / 4) + ks * 4 + (rem >> 3) * 2 + (rem & 1);
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
// One acquire load in flight per block, on one counter. Measured alternatives, all slower by 0.4 to 1 us per
// barrier: several polls in flight (acquire loads do not overlap: each holds back the loads behind it; relaxed
// loads with a fence after the last pay for the fence, and more polls queue on the counter's line with the
// arrivals), and arrivals spread over four counters on lines of their own.
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
                                          const int* token_rows,
                                          float* resid, const float* ln_w, float eps, unsigned char* xs,
                                          int row_bytes) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n4 = H / 4;                                    // float4 groups per row (H is a multiple of 8)
  for (int r = warp; r < T; r += kFuWarps) {               // rows beyond T feed accumulator rows nobody reads
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(xs + (size_t)r * row_bytes);
    const __nv_bfloat16* erow = embedding ? embedding + (size_t)token_ids[token_rows ? token_rows[r] : r] * H : nullptr;
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
    // The columns between H and the end of the last 32-wide chunk are multiplied too (by the packed matrices'
    // zero padding): they must hold zeros, not what an earlier phase left there (a NaN pattern times zero is NaN).
    const int kpad = (H + 31) / 32 * 32;
    if (lane < (kpad - H) / 8) *reinterpret_cast<uint4*>(dst + H + lane * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
}

// ---- The weight ring ---------------------------------------------------------------------------------------
// A TILE is what one stage holds: chunks [c0, c0 + nc) of one group of 8 weight rows, and for the projections
// whose epilogue needs two rows per output (a rotation pair of q/k/v; a gate row and its up row) the same
// chunks of the partner group behind it. A UNIT is a row group (with its partner) over all of K: one tile, or
// several when K does not fit a stage. Block b owns units b, b + grid, ... of every projection. Its tiles of
// the whole launch form one sequence (layer by layer: QKV, output, gate/up, down; unit by unit; K part by K
// part); tile i lives in stage i % nst and completes phase (i / nst) & 1 of that stage's barrier. Tile
// i + nst is asked for by the thread that knows tile i has been used up.
struct FuTileDesc;
struct FuRing {
  uint32_t base, bars;             // shared addresses of stage 0 and of its barrier
  int stage_bytes, nst;
  int cpt_pair, cpt_single;        // chunks per tile, with and without a partner group
  int ch_h, ch_q, ch_i;            // chunks in a row of H, nh D and I columns
  int nq, kq, no, ko, ng, kg, nd, kd;   // this block's units per projection, and tiles per unit
  int ng_ring;                     // gate/up units that go through the ring (all, or all but the last: see fu_overlay_issue)
  uint32_t ov_base, ov_bar;        // the overlay stage and its barrier; ov_base == 0: none
  int per_layer, n_total;          // this block's tiles per layer and in the launch
  int* issued;                     // [nst] tiles asked for so far, per stage (for the drain on an early exit)
  const struct FuTileDesc* tiles;  // [min(per_layer, kFuMaxTiles)] this block's tiles of a layer, in shared memory
};

__device__ __forceinline__ int fu_units_of_block(int n_units) {
  return (int)blockIdx.x < n_units ? (n_units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
}

__device__ __forceinline__ FuRing fu_ring_setup(const FusedArgs& a, uint32_t base, uint32_t bars, int nst, int* issued,
                                                uint32_t ov_base, uint32_t ov_bar) {
  FuRing R;
  R.issued = issued;
  R.base = base;
  R.bars = bars;
  R.stage_bytes = a.stage_bytes;
  R.nst = nst;
  R.cpt_pair = a.stage_bytes / (2 * kFuChunkBytes);
  R.cpt_single = a.stage_bytes / kFuChunkBytes;
  R.ch_h = (a.H + 31) / 32;
  R.ch_q = (a.nh * a.D + 31) / 32;
  R.ch_i = (a.I + 31) / 32;
  R.nq = fu_units_of_block((a.nh + 2 * a.nkv) * (a.D / 16));
  R.no = fu_units_of_block((a.H + 7) / 8);
  R.ng = fu_units_of_block((a.I + 7) / 8);
  R.nd = R.no;
  R.kq = (R.ch_h + R.cpt_pair - 1) / R.cpt_pair;
  R.kg = R.kq;
  R.ko = (R.ch_q + R.cpt_single - 1) / R.cpt_single;
  R.kd = (R.ch_i + R.cpt_single - 1) / R.cpt_single;
  const bool overlay = ov_base != 0 && R.kg == 1 && R.ng >= 1;
  R.ov_base = overlay ? ov_base : 0;
  R.ov_bar = ov_bar;
  R.ng_ring = R.ng - (overlay ? 1 : 0);
  R.per_layer = R.nq * R.kq + R.no * R.ko + R.ng_ring * R.kg + R.nd * R.kd;
  R.n_total = R.per_layer * a.n_layers;
  return R;
}

// Tile r of a layer, for this block: which matrix, where its chunks start (in chunks of the packed copy),
// how many there are, and whether a partner group follows.
struct FuTileDesc {
  uint32_t chunk_a, chunk_b;       // first chunk of the group and of the partner group, counted from the matrix start
  uint16_t nc;
  uint8_t matrix;                  // 0 QKV, 1 output, 2 gate/up, 3 down
  uint8_t pair;
};
constexpr int kFuMaxTiles = 64;    // table entries; a block with more tiles per layer works the rest out each time

__device__ __forceinline__ FuTileDesc fu_tile_desc(const FusedArgs& a, const FuRing& R, int r) {
  const int b = blockIdx.x, grid = gridDim.x;
  FuTileDesc d;
  if (r < R.nq * R.kq) {
    const int j = r / R.kq, kp = r - j * R.kq, u = b + j * grid;
    const int per_head = a.D / 16, head = u / per_head;
    const int row_a = head * a.D + (u - head * per_head) * 8, c0 = kp * R.cpt_pair;
    d.nc = (uint16_t)min(R.cpt_pair, R.ch_h - c0);
    d.chunk_a = (uint32_t)(row_a >> 3) * R.ch_h + c0;
    d.chunk_b = (uint32_t)((row_a + a.D / 2) >> 3) * R.ch_h + c0;
    d.matrix = 0;
    d.pair = 1;
  } else if ((r -= R.nq * R.kq) < R.no * R.ko) {
    const int j = r / R.ko, kp = r - j * R.ko, u = b + j * grid, c0 = kp * R.cpt_single;
    d.nc = (uint16_t)min(R.cpt_single, R.ch_q - c0);
    d.chunk_a = d.chunk_b = (uint32_t)u * R.ch_q + c0;
    d.matrix = 1;
    d.pair = 0;
  } else if ((r -= R.no * R.ko) < R.ng_ring * R.kg) {
    const int j = r / R.kg, kp = r - j * R.kg, u = b + j * grid, c0 = kp * R.cpt_pair;
    d.nc = (uint16_t)min(R.cpt_pair, R.ch_h - c0);
    d.chunk_a = (uint32_t)u * R.ch_h + c0;
    d.chunk_b = (uint32_t)(a.I / 8 + u) * R.ch_h + c0;
    d.matrix = 2;
    d.pair = 1;
  } else {
    r -= R.ng_ring * R.kg;
    const int j = r / R.kd, kp = r - j * R.kd, u = b + j * grid, c0 = kp * R.cpt_single;
    d.nc = (uint16_t)min(R.cpt_single, R.ch_i - c0);
    d.chunk_a = d.chunk_b = (uint32_t)u * R.ch_i + c0;
    d.matrix = 3;
    d.pair = 0;
  }
  return d;
}

// Ask for tile i (one thread). The caller knows that the stage is free.
__device__ __forceinline__ void fu_tile_issue(const FusedArgs& a, const FuRing& R, const FusedLayer* layers, int i) {
  if (i >= R.n_total) return;
  const int l = i / R.per_layer, r = i - l * R.per_layer;
  const FuTileDesc d = r < kFuMaxTiles ? R.tiles[r] : fu_tile_desc(a, R, r);
  const FusedLayer& L = layers[l];
  const __nv_bfloat16* W = d.matrix == 0 ? L.w_qkv : d.matrix == 1 ? L.w_o : d.matrix == 2 ? L.w_gu : L.w_down;
  const int s = i % R.nst;
  *reinterpret_cast<volatile int*>(R.issued + s) = i / R.nst + 1;
  const uint32_t bar = R.bars + s * 8, dst = R.base + s * R.stage_bytes, bytes = (uint32_t)d.nc * kFuChunkBytes;
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(d.pair ? 2 * bytes : bytes) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(W + (size_t)d.chunk_a * kFuChunkElems), "r"(bytes), "r"(bar) : "memory");
  if (d.pair)
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst + bytes), "l"(W + (size_t)d.chunk_b * kFuChunkElems), "r"(bytes), "r"(bar) : "memory");
}

// The overlay stage. While a layer's attention, output projection and gate/up run, most of the staging area
// (sized for the down projection's input) lies idle; one more stage is laid over its upper part, and the
// block's LAST gate/up unit of each layer goes there instead of through the ring, asked for as soon as the
// previous layer's down projection has read its input. A block whose gate/up units outnumber the ring's
// stages would otherwise start its last unit only after the first one has freed a stage.
__device__ __forceinline__ void fu_overlay_issue(const FusedArgs& a, const FuRing& R, const FusedLayer* layers, int l) {
  if (!R.ov_base || l >= a.n_layers) return;
  const int u = (int)blockIdx.x + (R.ng - 1) * (int)gridDim.x;
  const __nv_bfloat16* W = layers[l].w_gu;
  const uint32_t bytes = (uint32_t)R.ch_h * kFuChunkBytes;
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(R.ov_bar), "r"(2 * bytes) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(R.ov_base), "l"(W + (size_t)u * R.ch_h * kFuChunkElems), "r"(bytes), "r"(R.ov_bar) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(R.ov_base + bytes), "l"(W + (size_t)(a.I / 8 + u) * R.ch_h * kFuChunkElems), "r"(bytes), "r"(R.ov_bar) : "memory");
}

// Wait until tile i has landed. When the wait runs out the error word is raised and the block goes on with
// whatever the stage holds (every address it forms is in bounds whatever the data), so that no thread leaves
// the common path and the synchronisations that follow still pair up; the next grid barrier ends the launch.
__device__ __forceinline__ void fu_bar_wait(const FusedArgs& a, uint32_t bar, uint32_t parity, int* s_ok) {
  for (uint32_t spins = 0; spins < kFuSpinLimit; ++spins) {
    uint32_t done;
    asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return;
    if (spins > 256) {
      if (*reinterpret_cast<volatile int*>(s_ok) == 0) return;       // already failed: do not wait again
      __nanosleep(20);
    }
  }
  atomicCAS(a.error, 0, 1000);
  *reinterpret_cast<volatile int*>(s_ok) = 0;
}
__device__ __forceinline__ void fu_tile_wait(const FusedArgs& a, const FuRing& R, int i, int* s_ok) {
  // A barrier's phase can be told from the one before or after it, not from one two away: a warp that
  // polled for tile i while the stage's barrier was still two phases back (tile i - 2 nst not landed yet;
  // it happens as soon as a block has more tiles to wait for at once than stages) would be told "complete"
  // at once. So the warp first waits until tile i has been asked for, which happens only after tile
  // i - nst was used up; from then on the barrier is in tile i's phase or past it.
  const int s = i % R.nst, round = i / R.nst + 1;
  const volatile int* issued = R.issued + s;
  for (uint32_t spins = 0; *issued < round; ++spins) {
    if (spins > kFuSpinLimit) {
      atomicCAS(a.error, 0, 2000);
      *reinterpret_cast<volatile int*>(s_ok) = 0;
      return;
    }
    if (spins > 64) {
      if (*reinterpret_cast<volatile int*>(s_ok) == 0) return;
      __nanosleep(20);
    }
  }
  fu_bar_wait(a, R.bars + s * 8, (uint32_t)(round - 1) & 1u, s_ok);
}

// ---- The projections ---------------------------------------------------------------------------------------
enum : int { FU_QKV = 0, FU_ADD_RESID = 1 };

// A projection whose units a block takes one at a time, all 8 warps on a tile, each with an eighth of the
// tile's chunks; the partial sums meet in shared memory in warp order, so the result does not depend on
// timing. FU_QKV: units of 8 rows and their 8 rotation partners; bias, rotation and the writes of q and of
// the cache slots follow on the sums. FU_ADD_RESID: units of 8 rows; the sums are added into the residual
// stream (each element has one owner, so the update is in place).
// `stage_src`: null when the block's shared memory already holds the input (the norm wrote it), else the
// [T, K] bfloat16 matrix other blocks wrote, brought in row by row with bulk copies that complete on
// `stage_bar` (phase parity `stage_parity`); rows beyond T stay as they are: they only feed accumulator rows
// nobody reads. `halves` (a block then has at most one unit, and all its tiles fit the ring at once): the
// input's 9 to 16 rows come in two passes of 8, so that the staging area stays as small as for 8 tokens and
// the ring keeps its stages; the unit's tiles are read twice and given back in the second pass.
template <int MODE>
__device__ __forceinline__ void fu_project(const FusedArgs& a, const FusedLayer& L, const FuRing& R,
                                           const FusedLayer* layers, int tile0, int n_mine, int kparts, int cpt,
                                           int n_chunks, int N, int K, const __nv_bfloat16* stage_src,
                                           uint32_t stage_bar, uint32_t stage_parity, unsigned char* xs,
                                           int row_bytes, float* red, int* s_ok, bool halves = false) {
  constexpr bool PAIR = MODE == FU_QKV;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned char* xrow = xs + (lane >> 2) * row_bytes + (lane & 3) * 16;
  // Only max(8, T) rows are staged; a fragment row beyond them repeats the row 8 below it and feeds an
  // accumulator row nobody reads.
  const size_t hi_off = (lane >> 2) + 8 < a.T ? (size_t)8 * row_bytes : 0;
  const int n_pass = halves ? 2 : 1;
  for (int j = 0; j < n_mine; ++j) {
    const int u = (int)blockIdx.x + j * (int)gridDim.x;
    for (int pass = 0; pass < n_pass; ++pass) {
    const int tok0 = halves ? 8 * pass : 0;                        // first token of this pass
    const int n_tok = halves ? min(8, a.T - tok0) : a.T;           // tokens of this pass
    const size_t hi = halves ? 0 : hi_off;
    if (stage_src && (j == 0 || halves)) {
      // One bulk copy per token row (warp 0 asks; everybody waits on the staging barrier below). The columns
      // between K and the end of the last chunk are not part of the copy: they are zeroed by hand, since
      // whatever they hold is multiplied (by the packed matrix's zero padding).
      const int kpad = n_chunks * 32;
      if (warp == 0) {
        if (lane == 0) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // earlier plain accesses to the rows come first
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(stage_bar), "r"(n_tok * K * 2) : "memory");
        }
        __syncwarp();
        if (lane < n_tok)
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(smem_u32(xs) + lane * row_bytes), "l"(stage_src + (size_t)(tok0 + lane) * K), "r"(K * 2), "r"(stage_bar) : "memory");
      }
      if (kpad != K) {
        const int pieces = (kpad - K) / 8;
        for (int idx = tid; idx < n_tok * pieces; idx += kFuThreads) {
          const int r = idx / pieces, pc = idx - r * pieces;
          *reinterpret_cast<uint4*>(xs + (size_t)r * row_bytes + (size_t)(K + pc * 8) * 2) = make_uint4(0u, 0u, 0u, 0u);
        }
        __syncthreads();
      }
    }
    // What this thread's epilogue will need from global memory, asked for before the products so that the
    // round trips run beside them: the residual element it adds to; for q/k/v the bias pair, the token's
    // rotation pair and its cache slot.
    float resid_in = 0.f;
    if (!PAIR && tid < n_tok * 8) {
      const int n = u * 8 + (tid & 7);
      if (n < N) resid_in = __ldcg(a.resid + (size_t)(tok0 + (tid >> 3)) * N + n);
    }
    float e_b1 = 0.f, e_b2 = 0.f, e_cs = 1.f, e_sn = 0.f;
    int e_slot = -1;
    if (PAIR && tid < n_tok * 8) {
      const int tok = tid >> 3, f = tid & 7;
      const int per_head = a.D / 16, half = a.D / 2;
      const int head = u / per_head, i = (u - head * per_head) * 8 + f;
      if (L.b_qkv) {
        e_b1 = L.b_qkv[head * a.D + i];
        e_b2 = L.b_qkv[head * a.D + i + half];
      }
      if (head < a.nh + a.nkv) {
        int pos = a.positions[tok];
        if (pos < 0 || pos >= a.n_pos) {                   // never read outside the tables; tell the host
          atomicCAS(a.error, 0, 31);
          pos = pos < 0 ? 0 : a.n_pos - 1;
        }
        e_cs = a.cos_t[(size_t)pos * half + i];
        e_sn = a.sin_t[(size_t)pos * half + i];
      }
      if (head >= a.nh) e_slot = a.slot_map[tok];
    }
    // Two accumulator sets per row group, for even and odd chunks: the tensor-core pipeline then has two
    // independent chains to work on; they are added at the end.
    float acc_a[4] = {0.f, 0.f, 0.f, 0.f}, acc_b[4] = {0.f, 0.f, 0.f, 0.f};
    float acc_a2[4] = {0.f, 0.f, 0.f, 0.f}, acc_b2[4] = {0.f, 0.f, 0.f, 0.f};
    for (int kp = 0; kp < kparts; ++kp) {
      const int i = tile0 + j * kparts + kp;
      fu_tile_wait(a, R, i, s_ok);
      const int c0 = kp * cpt, nc = min(cpt, n_chunks - c0), per = (nc + kFuWarps - 1) / kFuWarps;
      const int w0 = warp * per, w1 = min(nc, w0 + per);
      if (stage_src && (j == 0 || halves) && kp == 0) {    // the staged input is needed only now
        fu_bar_wait(a, stage_bar, (stage_parity + (uint32_t)pass) & 1u, s_ok);
      }
      const uint32_t st = R.base + (i % R.nst) * R.stage_bytes + lane * 16;
      auto chunk = [&](int c, float (&da)[4], float (&db)[4]) {
        const uint4 wa = fu_lds128(st + c * kFuChunkBytes);
        const uint4 lo = *reinterpret_cast<const uint4*>(xrow + (c0 + c) * 64);
        const uint4 hv = hi ? *reinterpret_cast<const uint4*>(xrow + hi + (c0 + c) * 64) : lo;
        fu_mma(da, lo.x, hv.x, lo.y, hv.y, wa.x, wa.y);
        fu_mma(da, lo.z, hv.z, lo.w, hv.w, wa.z, wa.w);
        if (PAIR) {
          const uint4 wb = fu_lds128(st + (nc + c) * kFuChunkBytes);
          fu_mma(db, lo.x, hv.x, lo.y, hv.y, wb.x, wb.y);
          fu_mma(db, lo.z, hv.z, lo.w, hv.w, wb.z, wb.w);
        }
      };
      int c = w0;
#pragma unroll 2
      for (; c + 1 < w1; c += 2) {
        chunk(c, acc_a, acc_b);
        chunk(c + 1, acc_a2, acc_b2);
      }
      if (c < w1) chunk(c, acc_a, acc_b);
      if (kp + 1 < kparts && pass == n_pass - 1) {         // the stage is free once every warp is through
        __syncthreads();
        if (tid == 0) fu_tile_issue(a, R, layers, i + R.nst);
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      acc_a[e] += acc_a2[e];
      acc_b[e] += acc_b2[e];
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
    if (tid == 0 && pass == n_pass - 1) fu_tile_issue(a, R, layers, tile0 + j * kparts + kparts - 1 + R.nst);
    auto total = [&](int grp, int tok, int f) -> float {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kFuWarps; ++w) sum += red[(((size_t)w * 2 + grp) * 16 + tok) * 8 + f];
      return sum;
    };
    for (int idx = tid; idx < n_tok * 8; idx += kFuThreads) {
      const int tok = idx >> 3, f = idx & 7;
      if (MODE == FU_QKV) {
        const int per_head = a.D / 16, half = a.D / 2;
        const int head = u / per_head, i = (u - head * per_head) * 8 + f;
        const float x1 = total(0, tok, f) + e_b1, x2 = total(1, tok, f) + e_b2;     // (idx == tid: one pass)
        float o1 = x1, o2 = x2;
        if (head < a.nh + a.nkv) {
          o1 = __fadd_rn(__fmul_rn(x1, e_cs), __fmul_rn(-x2, e_sn));
          o2 = __fadd_rn(__fmul_rn(x2, e_cs), __fmul_rn(x1, e_sn));
        }
        __nv_bfloat16* dst = nullptr;
        if (head < a.nh) {
          // q goes to the attention phase in the order its tensor-core fragments are read (fu_q_index)
          __nv_bfloat16* qrow = a.q + ((size_t)tok * a.nh + head) * a.D;
          qrow[fu_q_index(i, a.D)] = __float2bfloat16_rn(o1);
          qrow[fu_q_index(i + half, a.D)] = __float2bfloat16_rn(o2);
        } else if (e_slot >= 0) {
          const bool is_k = head < a.nh + a.nkv;
          dst = (is_k ? L.kcache : L.vcache) + ((size_t)e_slot * a.nkv + (is_k ? head - a.nh : head - a.nh - a.nkv)) * a.D;
        }
        if (dst) {
          dst[i] = __float2bfloat16_rn(o1);
          dst[i + half] = __float2bfloat16_rn(o2);
        }
      } else {
        const int n = u * 8 + f;
        const size_t at = (size_t)(tok0 + tok) * N + n;
        if (n < N) a.resid[at] = (idx == tid ? resid_in : __ldcg(a.resid + at)) + total(0, tok, f);
      }
    }
    __syncthreads();   // `red` (and with `halves` the staged rows) are reused by what follows
    }
  }
}

// The gate/up projection with SwiGLU: one WARP owns a unit of 8 gate rows and their 8 up rows over the whole K
// range, so there is no partial sum to meet in shared memory and no block-wide synchronisation; the
// activation is computed on the accumulator registers, and the warp itself asks for the tile that follows
// into the stage it has used up.
__device__ __forceinline__ void fu_gate_up(const FusedArgs& a, const FuRing& R, const FusedLayer* layers, int tile0,
                                           int layer, const unsigned char* xs, int row_bytes, int* s_ok) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t2 = (lane & 3) * 2;
  const unsigned char* xrow = xs + g * row_bytes + (lane & 3) * 16;
  const size_t hi_off = (lane >> 2) + 8 < a.T ? (size_t)8 * row_bytes : 0;
  for (int j = warp; j < R.ng; j += kFuWarps) {
    const int u = (int)blockIdx.x + j * (int)gridDim.x;
    float acc_a[4] = {0.f, 0.f, 0.f, 0.f}, acc_b[4] = {0.f, 0.f, 0.f, 0.f};       // even chunks
    float acc_a2[4] = {0.f, 0.f, 0.f, 0.f}, acc_b2[4] = {0.f, 0.f, 0.f, 0.f};     // odd chunks
    const bool overlay = R.ov_base != 0 && j == R.ng - 1;    // (then R.kg == 1)
    for (int kp = 0; kp < R.kg; ++kp) {
      const int i = tile0 + j * R.kg + kp;
      if (overlay) fu_bar_wait(a, R.ov_bar, (uint32_t)layer & 1u, s_ok);
      else fu_tile_wait(a, R, i, s_ok);
      const int c0 = kp * R.cpt_pair, nc = min(R.cpt_pair, R.ch_h - c0);
      const uint32_t st = (overlay ? R.ov_base : R.base + (i % R.nst) * R.stage_bytes) + lane * 16;
      auto chunk = [&](int c, float (&da)[4], float (&db)[4]) {
        const uint4 wa = fu_lds128(st + c * kFuChunkBytes);
        const uint4 wb = fu_lds128(st + (nc + c) * kFuChunkBytes);
        const uint4 lo = *reinterpret_cast<const uint4*>(xrow + (c0 + c) * 64);
        const uint4 hi = hi_off ? *reinterpret_cast<const uint4*>(xrow + hi_off + (c0 + c) * 64) : lo;
        fu_mma(da, lo.x, hi.x, lo.y, hi.y, wa.x, wa.y);
        fu_mma(da, lo.z, hi.z, lo.w, hi.w, wa.z, wa.w);
        fu_mma(db, lo.x, hi.x, lo.y, hi.y, wb.x, wb.y);
        fu_mma(db, lo.z, hi.z, lo.w, hi.w, wb.z, wb.w);
      };
      int c = 0;
#pragma unroll 2
      for (; c + 1 < nc; c += 2) {
        chunk(c, acc_a, acc_b);
        chunk(c + 1, acc_a2, acc_b2);
      }
      if (c < nc) chunk(c, acc_a, acc_b);
      __syncwarp();                                        // every lane has its fragments: the stage is free
      if (lane == 0 && !overlay) fu_tile_issue(a, R, layers, i + R.nst);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      acc_a[e] += acc_a2[e];
      acc_b[e] += acc_b2[e];
    }
    // Accumulator layout: [0], [1] = token g, features t2, t2 + 1; [2], [3] = token g + 8, same features.
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int t = g + hh * 8;
      if (t >= a.T) continue;
      const float g0 = acc_a[2 * hh], g1 = acc_a[2 * hh + 1], u0 = acc_b[2 * hh], u1 = acc_b[2 * hh + 1];
      const int n = u * 8 + t2;
      if (n + 1 < a.I) {
        *reinterpret_cast<uint32_t*>(a.act + (size_t)t * a.I + n) =
            pack_bf16(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
      } else if (n < a.I) {
        a.act[(size_t)t * a.I + n] = __float2bfloat16_rn(g0 / (1.0f + expf(-g0)) * u0);
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

// Attention's working memory (the staging area of the projections): at least 16 keys per warp in flight, and
// room for the 8 warps' states.
template <int D> constexpr int fu_attn_min_bytes() {
  return kFuWarps * 16 * (D + 2) * 4 > kFuWarps * 16 * 4 * D ? kFuWarps * 16 * (D + 2) * 4 : kFuWarps * 16 * 4 * D;
}

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

    const int p_r0 = r0 < t.n_rows ? t.before + r0 / G : -1, p_r1 = r1 < t.n_rows ? t.before + r1 / G : -1;
    const int lo_r0 = a.window > 0 ? max(0, p_r0 - a.window + 1) : 0;
    const int lo_r1 = a.window > 0 ? max(0, p_r1 - a.window + 1) : 0;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // running max (log2 units) and sum per row
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    uint32_t qa[KS][4];
    bool q_loaded = false;
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
      if (!q_loaded) {                                     // the query fragments: asked for behind the copies, needed after them
        q_loaded = true;
        const int t4 = (lane & 3) * (D / 4);                 // this lane's block of a (permuted) query row
        const uint4* qr0 = nullptr;
        const uint4* qr1 = nullptr;
        if (r0 < t.n_rows)
          qr0 = reinterpret_cast<const uint4*>(a.q + ((size_t)(t.q_start + r0 / G) * a.nh + t.kvh * G + r0 % G) * D + t4);
        if (r1 < t.n_rows)
          qr1 = reinterpret_cast<const uint4*>(a.q + ((size_t)(t.q_start + r1 / G) * a.nh + t.kvh * G + r1 % G) * D + t4);
#pragma unroll
        for (int kk = 0; kk < KS / 2; ++kk) {                // 16 bytes hold two steps: [ks][0,1 | 8,9]
          const uint4 v0 = qr0 ? __ldcg(qr0 + kk) : make_uint4(0u, 0u, 0u, 0u);
          const uint4 v1 = qr1 ? __ldcg(qr1 + kk) : make_uint4(0u, 0u, 0u, 0u);
          qa[2 * kk][0] = v0.x; qa[2 * kk][2] = v0.y; qa[2 * kk + 1][0] = v0.z; qa[2 * kk + 1][2] = v0.w;
          qa[2 * kk][1] = v1.x; qa[2 * kk][3] = v1.y; qa[2 * kk + 1][1] = v1.z; qa[2 * kk + 1][3] = v1.w;
        }
      }
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
          for (int zb = z0; zb <= z1; zb += 8) {
            // Eight splits' loads are in flight before the first is used (past the end: the last split again,
            // left out of the sum).
            float2 ml[8];
            float4 pa[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int zz = min(zb + i, z1);
              ml[i] = __ldcg(reinterpret_cast<const float2*>(a.part_ml + (orow * a.max_splits + zz) * 2));
              pa[i] = __ldcg(reinterpret_cast<const float4*>(a.part_acc + (orow * a.max_splits + zz) * D + d));
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (zb + i > z1) break;
              const float m_new = fmaxf(mx, ml[i].x);
              const float keep = mx == -INFINITY ? 0.f : expf(mx - m_new);
              const float w = ml[i].x == -INFINITY ? 0.f : expf(ml[i].x - m_new);
              lsum = lsum * keep + ml[i].y * w;
              acc[0] = acc[0] * keep + pa[i].x * w;
              acc[1] = acc[1] * keep + pa[i].y * w;
              acc[2] = acc[2] * keep + pa[i].z * w;
              acc[3] = acc[3] * keep + pa[i].w * w;
              mx = m_new;
            }
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
  __shared__ __align__(8) unsigned long long s_full[kFuMaxStages + 2];   // the stages' barriers, the staging barrier, the overlay's
  __shared__ int s_issued[kFuMaxStages];
  __shared__ FuTileDesc s_tiles[kFuMaxTiles];
  __shared__ FusedLayer s_layers[kFuMaxLayers];
  // The requests' lengths, and the cache slots of this block's first attention unit, are the same in every
  // layer: look them up once, so that each layer can ask for its keys and values a phase before it reads
  // them and starts its copies without a table lookup.
  __shared__ int s_cu_q[17], s_before[16];
  __shared__ int s_slot[kFuWarps][kFuKeyCap];
  const int kmax = max(a.H, max(a.nh * a.D, a.I));
  const int rows = a.T > 8 ? a.T : 8;                                 // staged rows
  const int xs_bytes = a.halves ? max(8 * fu_row_bytes(kmax), rows * max(fu_row_bytes(a.H), fu_row_bytes(a.nh * a.D)))
                                : rows * fu_row_bytes(kmax);
  const int red_bytes = kFuWarps * 2 * 16 * 8 * (int)sizeof(float);
  unsigned char* xs = smem;                                          // staged inputs; attention's working memory
  float* red = reinterpret_cast<float*>(smem + xs_bytes);            // [8 warps][2 row groups][16][8]
  const int work_bytes = max(xs_bytes + red_bytes, fu_attn_min_bytes<D>());
  const int ring_off = (work_bytes + 127) / 128 * 128;
  const int nst = min(kFuMaxStages, (a.smem_bytes - ring_off) / a.stage_bytes);
  // The overlay stage lies in the staging area, above what attention and the narrower projections use of it.
  const int ov_off = (max(fu_attn_min_bytes<D>(), rows * max(fu_row_bytes(a.H), fu_row_bytes(a.nh * a.D))) + 127) / 128 * 128;
  const bool ov_fits = ov_off + a.stage_bytes <= xs_bytes;
  FuRing R = fu_ring_setup(a, smem_u32(smem + ring_off), smem_u32(s_full), nst, s_issued,
                           ov_fits ? smem_u32(smem + ov_off) : 0u, smem_u32(&s_full[kFuMaxStages + 1]));
  R.tiles = s_tiles;
  const int attn_bytes = R.ov_base ? ov_off : work_bytes;   // attention's working memory ends where the overlay begins
  const int rb_h = fu_row_bytes(a.H), rb_q = fu_row_bytes(a.nh * a.D), rb_i = fu_row_bytes(a.I);
  unsigned k = 0;
  bool ok = true;
  const uint32_t stage_bar = smem_u32(&s_full[kFuMaxStages]);
  uint32_t n_staged = 0;                      // uses of the staging barrier so far (its phase parity)
  int ov_issued = 0;                          // tiles asked for into the overlay stage so far

  // (The kernel behind this one, when it was launched as a programmatic dependent, may be scheduled as soon as
  // multiprocessors become free, and do what depends on nothing here, before this grid has drained: every block
  // of this grid is resident by now, so nothing can get in its way.)
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    s_ok = 1;
    for (int s = 0; s < kFuMaxStages; ++s) s_issued[s] = 0;
    for (int s = 0; s < nst; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(R.bars + s * 8));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_full[kFuMaxStages])));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_full[kFuMaxStages + 1])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i < a.n_layers * (int)(sizeof(FusedLayer) / sizeof(void*)); i += kFuThreads)
    reinterpret_cast<const void**>(s_layers)[i] = reinterpret_cast<const void* const*>(a.layers)[i];
  if ((int)threadIdx.x < min(R.per_layer, kFuMaxTiles)) s_tiles[threadIdx.x] = fu_tile_desc(a, R, threadIdx.x);
  if (threadIdx.x <= a.S) s_cu_q[threadIdx.x] = a.cu_q[threadIdx.x];
  if (threadIdx.x < a.S) s_before[threadIdx.x] = a.kv_before[threadIdx.x];
  __syncthreads();
  if (threadIdx.x == 0)
  {
    for (int i = 0; i < nst; ++i) fu_tile_issue(a, R, s_layers, i);
    fu_overlay_issue(a, R, s_layers, 0);
  }
  if (R.ov_base && a.n_layers > 0) ov_issued = 1;
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
    const FusedLayer& L = s_layers[l];
    const int t_qkv = l * R.per_layer, t_o = t_qkv + R.nq * R.kq, t_gu = t_o + R.no * R.ko, t_down = t_gu + R.ng_ring * R.kg;
    fu_stamp(a, l * 16 + 0);
    if (l + 1 < a.n_layers) {
      // The next layer's norm weights and bias are a few KB that nobody has touched in this launch: ask for them
      // now, so that a layer from now they come from the L2 and not from memory.
      const FusedLayer& N = s_layers[l + 1];
      const int lines_h = (a.H * 4 + 127) / 128, lines_b = N.b_qkv ? ((a.nh + 2 * a.nkv) * a.D * 4 + 127) / 128 : 0;
      for (int i = threadIdx.x; i < 2 * lines_h + lines_b; i += kFuThreads) {
        const char* p = i < lines_h ? (const char*)N.ln1_w + (size_t)i * 128
                        : i < 2 * lines_h ? (const char*)N.ln2_w + (size_t)(i - lines_h) * 128
                                          : (const char*)N.b_qkv + (size_t)(i - 2 * lines_h) * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
      }
    }
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
    fu_norm_rows(a.T, a.H, l == 0 ? a.embedding : nullptr, a.token_ids, a.token_rows, a.resid, L.ln1_w, a.eps1, xs,
                 rb_h);
    __syncthreads();
    fu_stamp(a, l * 16 + 1);
    fu_project<FU_QKV>(a, L, R, s_layers, t_qkv, R.nq, R.kq, R.cpt_pair, R.ch_h, (a.nh + 2 * a.nkv) * a.D, a.H, nullptr,
                       0, 0, xs, rb_h, red, &s_ok);
    fu_stamp(a, l * 16 + 2);
    if (!(ok = fu_grid_sync(a, k, &s_ok))) break;
    fu_stamp(a, l * 16 + 3);
    // B: attention (its working memory is the staging area; the ring's stages stay untouched)
    fu_attention<D>(a, L, xs, attn_bytes, s_cu_q, s_before, s_slot, l);
    fu_stamp(a, l * 16 + 4);
    if (!(ok = fu_grid_sync(a, k, &s_ok))) break;
    fu_stamp(a, l * 16 + 5);
    // C: output projection; then D: norm + gate/up + SwiGLU, and E: down projection. The two projections that add
    // into the stream share ONE copy of their code (a loop of two that is not unrolled): the kernel's instructions
    // (190 KB with a copy each) are more than a multiprocessor's instruction cache holds, every layer walks through
    // all of them, and 24 KB less made every phase a little faster (29.9 -> 29.1 us a layer at batch 8).
    bool left = false;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      if (which == 1) {
        fu_norm_rows(a.T, a.H, nullptr, a.token_ids, nullptr, a.resid, L.ln2_w, a.eps2, xs, rb_h);
        __syncthreads();
        fu_stamp(a, l * 16 + 7);
        fu_gate_up(a, R, s_layers, t_gu, l, xs, rb_h, &s_ok);
        fu_stamp(a, l * 16 + 8);
        if (!(ok = fu_grid_sync(a, k, &s_ok))) { left = true; break; }
      }
      const bool down = which == 1;
      fu_project<FU_ADD_RESID>(a, L, R, s_layers, down ? t_down : t_o, down ? R.nd : R.no, down ? R.kd : R.ko, R.cpt_single,
                               down ? R.ch_i : R.ch_q, a.H, down ? a.I : a.nh * a.D, down ? a.act : a.attn, stage_bar,
                               n_staged & 1u, xs, down ? rb_i : rb_q, red, &s_ok, down && a.halves != 0);
      if ((down ? R.nd : R.no) > 0) n_staged += (down && a.halves) ? 2 : 1;
      if (!down) {
        fu_stamp(a, l * 16 + 6);
        if (!(ok = fu_grid_sync(a, k, &s_ok))) { left = true; break; }
      }
    }
    if (left) break;
    if (threadIdx.x == 0) fu_overlay_issue(a, R, s_layers, l + 1);   // the staging area has been read: it is free again
    if (R.ov_base && l + 1 < a.n_layers) ov_issued = l + 2;
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
  } else {
    // Leaving early: copies may still be on their way into this block's shared memory. Give each stage's
    // barrier a bounded chance to complete its current phase (either parity counts) before the block ends.
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int s = 0; s <= nst + 1; ++s) {                 // the stages, the staging barrier, the overlay's
        const int issued = s < nst ? s_issued[s] : s == nst ? (int)n_staged : ov_issued;
        if (!issued) continue;
        const uint32_t bar = s < nst ? R.bars + s * 8 : s == nst ? stage_bar : R.ov_bar;
        const uint32_t parity = (uint32_t)(issued - 1) & 1u;
        for (uint32_t spins = 0; spins < (1u << 20); ++spins) {
          uint32_t done;
          asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                       : "=r"(done) : "r"(bar), "r"(parity) : "memory");
          if (done) break;
          __nanosleep(100);
        }
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

static int fu_host_row_bytes(int K) {           // fu_row_bytes for the host
  const int kpad = (K + 31) / 32 * 32;
  return kpad * 2 + ((64 - (kpad * 2) % 128) + 128) % 128;
}

// How a step of T tokens is laid out in the block's shared memory: the bytes of a ring stage and whether the
// down projection's input comes in two passes of 8 rows. False when the sizes leave no room for a ring stage
// beside the staged activations (wide models at many tokens): such steps are not for this kernel.
template <int D>
bool fu_plan(int H, int nh, int I, int T, int n_sm, int smem, int* stage_bytes_out, bool* halves_out) {
  const int rb_h = fu_host_row_bytes(H), rb_q = fu_host_row_bytes(nh * D), rb_i = fu_host_row_bytes(I);
  const int rb_narrow = rb_h > rb_q ? rb_h : rb_q, rb_max = rb_narrow > rb_i ? rb_narrow : rb_i;
  const int red_bytes = kFuWarps * 2 * 16 * 8 * (int)sizeof(float);
  // A stage holds a row group and its partner over all of H when that fits 32 KB, else 32 KB worth of chunks.
  const int ch_h = (H + 31) / 32;
  const int stage_bytes = 2 * ch_h * 512 <= 32768 ? 2 * ch_h * 512 : 32768;
  auto ring_offset = [&](int xs_bytes) {      // the staging area doubles as attention's working memory
    const int work = xs_bytes + red_bytes > fu_attn_min_bytes<D>() ? xs_bytes + red_bytes : fu_attn_min_bytes<D>();
    return (work + 127) / 128 * 128;
  };
  const int rows = T > 8 ? T : 8;
  // Steps of 9 to 16 tokens: the down projection's input (T rows of I columns) would take the room of most
  // ring stages. Where every block has at most one down-projection unit and the unit's tiles all fit the ring
  // at once, the input comes in two passes of 8 rows instead and the staging area stays as for 8 tokens.
  const int xs_halves = 8 * rb_max > rows * rb_narrow ? 8 * rb_max : rows * rb_narrow;
  int nst_halves = (smem - ring_offset(xs_halves)) / stage_bytes;
  if (nst_halves > kFuMaxStages) nst_halves = kFuMaxStages;
  const int cpt_single = stage_bytes / 512, kd = ((I + 31) / 32 + cpt_single - 1) / cpt_single;
  const int nst_rows = (smem - ring_offset(rows * rb_max)) / stage_bytes;
  // (Measured at the 0.5B sizes: with two or more stages left, staging all rows in one pass is as fast or faster.)
  const bool halves = T > 8 && nst_rows <= 1 && (H + 7) / 8 <= n_sm && kd <= nst_halves;
  const int xs_bytes = halves ? xs_halves : rows * rb_max;
  if (ring_offset(xs_bytes) + stage_bytes > smem) return false;
  *stage_bytes_out = stage_bytes;
  *halves_out = halves;
  return true;
}

template <int D>
int launch_decode_fused(const FusedArgs& a, cudaStream_t stream) {
  auto kern = decode_fused_kernel<D>;
  constexpr int smem = 212 * 1024;
  static int n_sm = 0, per_sm = 0;
  if (!n_sm) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kFuThreads, smem);
    if (e != cudaSuccess || per_sm < 1) {
      n_sm = 0;
      return e != cudaSuccess ? (int)e : TM_ERR_UNSUPPORTED_SHAPE;
    }
  }
  int stage_bytes = 0;
  bool halves = false;
  if (!fu_plan<D>(a.H, a.nh, a.I, a.T, n_sm, smem, &stage_bytes, &halves) || a.n_layers > kFuMaxLayers)
    return TM_ERR_UNSUPPORTED_SHAPE;
  FusedArgs args = a;
  args.smem_bytes = smem;
  args.stage_bytes = stage_bytes;
  args.halves = halves ? 1 : 0;
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

// The largest number of tokens (0 to 16) a step of these sizes may have for tm_decode_fused: every count up to
// it has room in shared memory for its staged activations and at least one ring stage. `n_sm`: the device's SMs.
extern "C" int tm_decode_fused_max_tokens(int H, int nh, int nkv, int D, int I, int n_sm) {
  if (H % 8 || I % 8 || (nh * D) % 8 || nkv <= 0 || nh % nkv || nh / nkv > 16 || (D != 64 && D != 128)) return 0;
  int best = 0, stage = 0;
  bool halves = false;
  for (int T = 1; T <= 16; ++T) {
    const bool ok = D == 64 ? tmk::fu_plan<64>(H, nh, I, T, n_sm, 212 * 1024, &stage, &halves)
                            : tmk::fu_plan<128>(H, nh, I, T, n_sm, 212 * 1024, &stage, &halves);
    if (!ok) break;
    best = T;
  }
  return best;
}

extern "C" int tm_decode_fused_args_size() { return (int)sizeof(tmk::FusedArgs); }
extern "C" int tm_decode_fused_layer_size() { return (int)sizeof(tmk::FusedLayer); }
