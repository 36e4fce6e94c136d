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
#include "attention_decode_core.cuh"

namespace tmk {

constexpr int kFuThreads = 256;
constexpr int kFuWarps = 8;
constexpr uint32_t kFuSpinLimit = 1u << 22;

struct FusedLayer {
  const float* ln1_w;
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
  unsigned long long* timing;      // null, or [n_layers * 10 + 1] nanosecond stamps written by block 0 (profiling aid)
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

__device__ __forceinline__ int fu_row_bytes(int K) {
  const int kpad = (K + 31) / 32 * 32;
  return kpad * 2 + ((64 - (kpad * 2) % 128) + 128) % 128;   // 64 mod 128: conflict-free fragment reads
}

// Grid-wide barrier number `k` (0-based) of this launch. Returns false when the wait ran out.
__device__ __forceinline__ bool fu_grid_sync(const FusedArgs& a, unsigned& k, int* s_ok) {
  __syncthreads();
  if (threadIdx.x == 0) {
    // Release-arrive and acquire-poll at device scope: the block's writes (ordered before by the block
    // barrier above) are visible to every block that sees the counter reach the target.
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(a.bar) : "memory");
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

// Copy a [T, K] bfloat16 matrix other blocks wrote into the staged layout (rows beyond T are left as they are:
// they only feed accumulator rows nobody reads).
__device__ __forceinline__ void fu_stage(const __nv_bfloat16* src, int T, int K, unsigned char* xs, int row_bytes) {
  const int chunks = ((K + 31) / 32 * 32) / 8;
  const uint32_t base = smem_u32(xs);
  for (int idx = threadIdx.x; idx < T * chunks; idx += kFuThreads) {
    const int r = idx / chunks, c = idx - r * chunks;
    const bool ok = c * 8 < K;
    cp_async16(base + r * row_bytes + c * 16, ok ? src + (size_t)r * K + c * 8 : src, ok);
  }
  cp_async_commit();
  cp_async_wait<0>();
}

// The weight-streaming product of gemm_skinny_bf16.cu for one block-sized unit at a time: `ng` groups of 8
// weight rows, K cut across the 8 / ng warps of a group, partial sums met in shared memory in warp order.
template <int MODE>
__device__ __forceinline__ void fu_gemm_units(const FusedArgs& a, const FusedLayer& L, const __nv_bfloat16* W, int N,
                                              int K, int ng, int n_units, const unsigned char* xs, int row_bytes,
                                              float* red, float* out_f32) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kw = kFuWarps / ng;
  const int g = warp / kw, kpart = warp - g * kw;
  const int n_chunks = (K + 31) / 32;
  const int per = (n_chunks + kw - 1) / kw;
  const int c_begin = kpart * per, c_end = min(n_chunks, c_begin + per);
  const unsigned char* xrow = xs + (lane >> 2) * row_bytes + (lane & 3) * 16;
  constexpr int U = 8;
  for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
    int row0;
    if (MODE == FU_QKV) {
      const int per_head = a.D / 16;
      const int head = u / per_head, i0 = (u - head * per_head) * 8;
      row0 = head * a.D + i0 + g * (a.D / 2);
    } else if (MODE == FU_SWIGLU) {
      row0 = u * 8 + g * a.I;
    } else {
      row0 = (u * ng + g) * 8;
    }
    const int wrow = row0 + (lane >> 2);
    const bool row_ok = wrow < N;
    const __nv_bfloat16* wp = W + (size_t)(row_ok ? wrow : 0) * K + (lane & 3) * 8;
    auto load_w = [&](int c) -> uint4 {
      const int k = c * 32 + (lane & 3) * 8;
      if (row_ok && c < c_end && k < K) return fu_ldg_stream(wp + c * 32);
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
          const uint4 hi = *reinterpret_cast<const uint4*>(xrow + (size_t)8 * row_bytes + (c + i) * 64);
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
    if (MODE == FU_QKV) {
      const int per_head = a.D / 16, half = a.D / 2;
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
    } else if (MODE == FU_SWIGLU) {
      for (int idx = tid; idx < a.T * 8; idx += kFuThreads) {
        const int t = idx >> 3, j = idx & 7, n = u * 8 + j;
        if (n >= a.I) continue;
        const float gt = total(t, 0, j), up = total(t, 1, j);
        a.act[(size_t)t * a.I + n] = __float2bfloat16_rn(gt / (1.0f + expf(-gt)) * up);
      }
    } else {
      const int feats = ng * 8;
      for (int idx = tid; idx < a.T * feats; idx += kFuThreads) {
        const int t = idx / feats, fj = idx - t * feats;
        const int n = (u * ng + (fj >> 3)) * 8 + (fj & 7);
        // residual + branch, in 32-bit; each element has one owner, so the update is in place
        if (n < N) out_f32[(size_t)t * N + n] = __ldcg(out_f32 + (size_t)t * N + n) + total(t, fj >> 3, fj & 7);
      }
    }
    __syncthreads();   // `red` is reused by the next unit
  }
}

// Projections whose epilogue needs two weight rows per output (a rotation pair of q/k/v, or a gate row and
// its up row): one WARP owns a unit of 8 + 8 rows over the whole K range, so there is no partial sum to meet
// in shared memory and no block-wide synchronisation; the epilogue runs on the accumulator registers.
template <int MODE>
__device__ __forceinline__ void fu_pair_units(const FusedArgs& a, const FusedLayer& L, const __nv_bfloat16* W, int N,
                                              int K, int n_units, const unsigned char* xs, int row_bytes) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t2 = (lane & 3) * 2;
  const int n_chunks = (K + 31) / 32;
  const unsigned char* xrow = xs + g * row_bytes + (lane & 3) * 16;
  constexpr int U = 6;
  // Unit u goes to warp (u / grid) of block (u % grid): consecutive units land on different SMs.
  for (int u = warp * gridDim.x + blockIdx.x; u < n_units; u += kFuWarps * gridDim.x) {
    int row_a, row_b, head = 0, i0 = 0;
    if (MODE == FU_QKV) {
      const int per_head = a.D / 16;
      head = u / per_head;
      i0 = (u - head * per_head) * 8;
      row_a = head * a.D + i0;
      row_b = row_a + a.D / 2;
    } else {
      row_a = u * 8;
      row_b = a.I + u * 8;
    }
    const bool ok_a = row_a + g < N && (MODE == FU_QKV || row_a + g < a.I), ok_b = row_b + g < N;
    const __nv_bfloat16* wa = W + (size_t)(ok_a ? row_a + g : 0) * K + (lane & 3) * 8;
    const __nv_bfloat16* wb = W + (size_t)(ok_b ? row_b + g : 0) * K + (lane & 3) * 8;
    auto load = [&](const __nv_bfloat16* p, bool ok, int c) -> uint4 {
      const int k = c * 32 + (lane & 3) * 8;
      if (ok && c < n_chunks && k < K) return fu_ldg_stream(p + c * 32);
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
          const uint4 hi = *reinterpret_cast<const uint4*>(xrow + (size_t)8 * row_bytes + (c + i) * 64);
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
      if (MODE == FU_SWIGLU) {
        const int n = u * 8 + t2;
        if (n + 1 < a.I) {
          *reinterpret_cast<uint32_t*>(a.act + (size_t)t * a.I + n) =
              pack_bf16(v1[0] / (1.0f + expf(-v1[0])) * v2[0], v1[1] / (1.0f + expf(-v1[1])) * v2[1]);
        } else if (n < a.I) {
          a.act[(size_t)t * a.I + n] = __float2bfloat16_rn(v1[0] / (1.0f + expf(-v1[0])) * v2[0]);
        }
      } else {
        const int half = a.D / 2, i = i0 + t2;
        const int c0 = head * a.D + i, c1 = c0 + half;
        if (L.b_qkv) {
          v1[0] += L.b_qkv[c0];
          v1[1] += L.b_qkv[c0 + 1];
          v2[0] += L.b_qkv[c1];
          v2[1] += L.b_qkv[c1 + 1];
        }
        float o1[2] = {v1[0], v1[1]}, o2[2] = {v2[0], v2[1]};
        if (head < a.nh + a.nkv) {
          int pos = a.positions[t];
          pos = pos < 0 ? 0 : (pos >= a.n_pos ? a.n_pos - 1 : pos);
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float cs = a.cos_t[(size_t)pos * half + i + e], sn = a.sin_t[(size_t)pos * half + i + e];
            o1[e] = __fadd_rn(__fmul_rn(v1[e], cs), __fmul_rn(-v2[e], sn));
            o2[e] = __fadd_rn(__fmul_rn(v2[e], cs), __fmul_rn(v1[e], sn));
          }
        }
        __nv_bfloat16* dst = nullptr;
        if (head < a.nh) {
          dst = a.q + ((size_t)t * a.nh + head) * a.D;
        } else {
          const int slot = a.slot_map[t];
          if (slot >= 0) {
            const bool is_k = head < a.nh + a.nkv;
            dst = (is_k ? L.kcache : L.vcache) + ((size_t)slot * a.nkv + (is_k ? head - a.nh : head - a.nh - a.nkv)) * a.D;
          }
        }
        if (dst) {
          *reinterpret_cast<uint32_t*>(dst + i) = pack_bf16(o1[0], o1[1]);
          *reinterpret_cast<uint32_t*>(dst + i + half) = pack_bf16(o2[0], o2[1]);
        }
      }
    }
  }
}

template <int D>
__device__ __forceinline__ void fu_attention(const FusedArgs& a, const FusedLayer& L, unsigned char* smem) {
  const int team = threadIdx.x >> 7, ttid = threadIdx.x & 127;
  unsigned char* tsmem = smem + (size_t)team * decode_unit_smem_bytes<D>();
  __shared__ int s_last[2];
  auto team_sync = [team] { asm volatile("bar.sync %0, 128;" ::"r"(team + 1) : "memory"); };
  const int G = a.nh / a.nkv;
  const int n_units = a.S * a.nkv * a.max_splits;
  for (int u = blockIdx.x * 2 + team; u < n_units; u += gridDim.x * 2) {
    const int z = u % a.max_splits;
    const int sk = u / a.max_splits;
    const int kvh = sk % a.nkv, s = sk / a.nkv;
    const int q_start = a.cu_q[s], q_len = a.cu_q[s + 1] - q_start, before = a.kv_before[s];
    const int* table = a.block_table + (size_t)s * a.bt_stride;
    const bool worked = decode_attention_unit<D>(a.q, L.kcache, L.vcache, table, q_start, q_len, before, kvh, z,
                                                 a.part_acc, a.part_ml, a.nh, a.nkv, a.page_size, a.scale_log2,
                                                 a.window, a.split_keys, a.max_splits, tsmem, ttid, team_sync);
    if (!worked) continue;                     // uniform over the team: every thread sees the same ranges
    // How many splits hold keys for this (request, kv head): the last one to finish merges them.
    const int n_rows = min(q_len * G, 16);
    const int p_min = before, p_max = before + (n_rows - 1) / G;
    const int j_lo = a.window > 0 ? max(0, p_min - a.window + 1) : 0;
    const int expected = p_max / a.split_keys - j_lo / a.split_keys + 1;
    __threadfence();
    team_sync();
    if (ttid == 0) s_last[team] = atomicAdd(&a.attn_count[s * a.nkv + kvh], 1) == expected - 1;
    team_sync();
    if (s_last[team]) {
      __threadfence();
      for (int idx = ttid; idx < n_rows * (D / 4); idx += 128) {
        const int r = idx / (D / 4), d = (idx - r * (D / 4)) * 4;
        const int tok = q_start + r / G, head = kvh * G + r % G;
        const size_t orow = (size_t)tok * a.nh + head;
        const int p = before + r / G;
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
        uint2 o;
        o.x = pack_bf16(acc[0] * inv, acc[1] * inv);
        o.y = pack_bf16(acc[2] * inv, acc[3] * inv);
        *reinterpret_cast<uint2*>(a.attn + orow * D + d) = o;
      }
      if (ttid == 0) a.attn_count[s * a.nkv + kvh] = 0;
    }
    team_sync();   // s_last and the team's shared memory are reused by the next unit
  }
}

template <int D>
__global__ void __launch_bounds__(kFuThreads, 1) decode_fused_kernel(const FusedArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  const int kmax = max(a.H, max(a.nh * a.D, a.I));
  const int xs_bytes = 16 * fu_row_bytes(kmax);
  unsigned char* xs = smem;
  float* red = reinterpret_cast<float*>(smem + xs_bytes);            // [8 warps][16][8]
  const int rb_h = fu_row_bytes(a.H), rb_q = fu_row_bytes(a.nh * a.D), rb_i = fu_row_bytes(a.I);
  unsigned k = 0;
  bool ok = true;
  const int qkv_rows = (a.nh + 2 * a.nkv) * a.D;
  __syncthreads();

  const size_t qkv_bytes = (size_t)qkv_rows * a.H * 2, o_bytes = (size_t)a.H * a.nh * a.D * 2;
  const size_t gu_bytes = (size_t)2 * a.I * a.H * 2, down_bytes = (size_t)a.H * a.I * 2;
  __shared__ FusedLayer s_layer[2];          // this layer's pointers and the next one's, fetched a phase early
  if (threadIdx.x == 0 && a.n_layers > 0) s_layer[0] = a.layers[0];
  // The cache slots of the first attention unit of each half block are the same in every layer: look them
  // up once, so that each layer can ask for its keys and values a phase before it reads them.
  __shared__ int s_kv_slot[2][kDecBN], s_kv_head[2];
  {
    const int team = threadIdx.x >> 7, ttid = threadIdx.x & 127;
    const int u = blockIdx.x * 2 + team;
    if (ttid < kDecBN) {
      int slot = -1;
      if (u < a.S * a.nkv * a.max_splits) {
        const int z = u % a.max_splits, sk = u / a.max_splits;
        const int kvh = sk % a.nkv, sq = sk / a.nkv;
        const int j = z * a.split_keys + ttid;
        if (ttid == 0) s_kv_head[team] = kvh;
        if (ttid < a.split_keys && j < a.kv_before[sq] + a.cu_q[sq + 1] - a.cu_q[sq]) {
          const int page = a.block_table[(size_t)sq * a.bt_stride + j / a.page_size];
          if (page >= 0) slot = page * a.page_size + j % a.page_size;
        }
      }
      s_kv_slot[team][ttid] = slot;
    }
  }
  __syncthreads();

  for (int l = 0; l < a.n_layers && ok; ++l) {
    const FusedLayer& L = s_layer[l & 1];
    fu_stamp(a, l * 10 + 0);
    fu_prefetch_l2(L.w_o, o_bytes);
    fu_prefetch_l2(L.w_gu, gu_bytes);
    {
      const int slot = s_kv_slot[threadIdx.x >> 7][(threadIdx.x & 127) >> 1];
      if (slot >= 0) {
        const __nv_bfloat16* p = ((threadIdx.x & 1) ? L.vcache : L.kcache) +
                                 ((size_t)slot * a.nkv + s_kv_head[threadIdx.x >> 7]) * D;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
        if (D > 64) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + 64));
      }
    }
    // A: norm + QKV
    fu_norm_rows(a.T, a.H, l == 0 ? a.embedding : nullptr, a.token_ids, a.resid, L.ln1_w, a.eps1, xs, rb_h);
    __syncthreads();
    fu_stamp(a, l * 10 + 1);
    fu_gemm_units<FU_QKV>(a, L, L.w_qkv, qkv_rows, a.H, 2, (a.nh + 2 * a.nkv) * (a.D / 16), xs, rb_h, red, nullptr);
    fu_stamp(a, l * 10 + 2);
    if (!(ok = fu_grid_sync(a, k, &s_ok))) break;
    fu_stamp(a, l * 10 + 3);
    // B: attention
    fu_attention<D>(a, L, smem);
    fu_stamp(a, l * 10 + 4);
    if (!(ok = fu_grid_sync(a, k, &s_ok))) break;
    fu_stamp(a, l * 10 + 5);
    // C: output projection
    fu_prefetch_l2(L.w_down, down_bytes);
    if (l + 1 < a.n_layers) {
      if (threadIdx.x == 0) s_layer[(l + 1) & 1] = a.layers[l + 1];
      fu_prefetch_l2(a.layers[l + 1].w_qkv, qkv_bytes);
    }
    fu_stage(a.attn, a.T, a.nh * a.D, xs, rb_q);
    __syncthreads();
    fu_gemm_units<FU_ADD_RESID>(a, L, L.w_o, a.H, a.nh * a.D, 1, (a.H + 7) / 8, xs, rb_q, red, a.resid);
    fu_stamp(a, l * 10 + 6);
    if (!(ok = fu_grid_sync(a, k, &s_ok))) break;
    // D: norm + gate/up + SwiGLU
    fu_norm_rows(a.T, a.H, nullptr, a.token_ids, a.resid, L.ln2_w, a.eps2, xs, rb_h);
    __syncthreads();
    fu_stamp(a, l * 10 + 7);
    fu_pair_units<FU_SWIGLU>(a, L, L.w_gu, 2 * a.I, a.H, (a.I + 7) / 8, xs, rb_h);
    fu_stamp(a, l * 10 + 8);
    if (!(ok = fu_grid_sync(a, k, &s_ok))) break;
    // E: down projection
    fu_stage(a.act, a.T, a.I, xs, rb_i);
    __syncthreads();
    fu_gemm_units<FU_ADD_RESID>(a, L, L.w_down, a.H, a.I, 1, (a.H + 7) / 8, xs, rb_i, red, a.resid);
    fu_stamp(a, l * 10 + 9);
    if (!(ok = fu_grid_sync(a, k, &s_ok))) break;
  }
  fu_stamp(a, a.n_layers * 10);

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
  int smem = 16 * row_bytes + kFuWarps * 16 * 8 * (int)sizeof(float);
  const int attn_bytes = 2 * decode_unit_smem_bytes<D>();
  if (attn_bytes > smem) smem = attn_bytes;
  if (smem > 220 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
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
      a.split_keys <= 0 || a.split_keys % tmk::kDecBN || a.max_splits <= 0 || !a.bar || !a.error)
    return TM_ERR_UNSUPPORTED_SHAPE;
  if (a.D == 64) return tmk::launch_decode_fused<64>(a, stream);
  if (a.D == 128) return tmk::launch_decode_fused<128>(a, stream);
  return TM_ERR_UNSUPPORTED_SHAPE;
}

extern "C" int tm_decode_fused_args_size() { return (int)sizeof(tmk::FusedArgs); }
extern "C" int tm_decode_fused_layer_size() { return (int)sizeof(tmk::FusedLayer); }
