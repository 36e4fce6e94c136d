// Prompt-step matrix products on the 5th-generation tensor cores: out = x[T, K] . W[N, K]^T, bfloat16
// operands, float32 accumulators in tensor memory, with the projection's own epilogue.
//
// One persistent block per SM, 8 warps with fixed roles:
//   warp 0   one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the 128 x 64
//            activation tile and two 128 x 64 weight tiles into a 4-stage shared-memory ring;
//   warp 1   one lane issues tcgen05.mma (M = 128 tokens, N = 256 weight rows, K = 16 per instruction,
//            operands straight from shared memory through matrix descriptors) into one of two 256-column
//            accumulators in tensor memory, and commits each stage back to the loader;
//   warp 2   allocates and frees the 512 columns of tensor memory;
//   warps 4-7 read a finished accumulator back with tcgen05.ld (each warp its own 32 lanes = 32 tokens)
//            and run the epilogue while the next tile's products already go into the other accumulator.
// Epilogues (the reference's projections, src/infer/model/layers.py:127-164):
//   STORE   out[t, n] bfloat16                                                    (o_proj, down_proj)
//   SWIGLU  the tile's 256 weight rows are 128 gate rows and the 128 matching up rows;
//           out[t, i] = silu(gate) * up, so the [T, 2I] product never exists in memory
//   QKV     + bias, rotate-half position encoding of q and k, q to q_out, k and v to their cache slots
// Every wait on an mbarrier is bounded: when it runs out, the block raises an error word, skips the
// rest of its work, still frees its tensor memory, and the host reports the failure.
#include <cuda.h>

#include "tcgen05_util.cuh"

namespace tmk {

// The tile is 128 tokens by BN weight rows: 256 where the projection has many tiles (gate/up, down, o_proj), 128
// where 256 would leave most SMs without a tile (the q/k/v projection of a 2,048-token prompt at 14 + 2 x 2
// heads of 64 has 80 tiles of 256 columns and 144 of 128: one wave that fills the chip).
constexpr int kT5BM = 128, kT5BK = 64;
constexpr int kT5ABytes = kT5BM * kT5BK * 2;            // 16 KB
template <int BN> constexpr int t5_b_bytes() { return BN * kT5BK * 2; }                       // 32, 16 or 8 KB
template <int BN> constexpr int t5_stage_bytes() { return kT5ABytes + t5_b_bytes<BN>(); }     // 48, 32 or 24 KB
template <int BN> constexpr int t5_stages() { return BN == 256 ? 4 : (BN == 128 ? 6 : 8); }
constexpr int kT5Threads = 256;
enum : int { T5_STORE = 0, T5_SWIGLU = 1, T5_QKV = 2, T5_ADD_F32 = 3 };

struct T5Args {
  int T, N, K, mode;
  int n_tiles_m, n_tiles_n;
  int n_splits, kb_per_split;   // the K range cut into n_splits pieces of kb_per_split blocks of 64 (1 piece: all of K)
  float* out_f32;           // ADD_F32: [T, N] float32 that the product is added into (one atomic add per piece)
  __nv_bfloat16* out;       // STORE: [T, N]; SWIGLU: [T, inter]
  int ldo, inter;
  // QKV
  const float* bias;
  const int* positions;
  const float* cos_t;
  const float* sin_t;
  const int* slot_map;
  __nv_bfloat16* q_out;
  __nv_bfloat16* kcache;
  __nv_bfloat16* vcache;
  int nh, nkv, D, n_pos;
  int* error;               // device word, 0 when all is well
  int pdl;                  // launched with programmatic dependent launch (a decode step's product)
};

// --- PTX wrappers (the rest are in tcgen05_util.cuh) -----------------------------------------------

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void store8_bf16(__nv_bfloat16* dst, const float* v) {
  uint4 o;
  o.x = ([](float a, float b) { __nv_bfloat162 t = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&t); })(v[0], v[1]);
  o.y = ([](float a, float b) { __nv_bfloat162 t = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&t); })(v[2], v[3]);
  o.z = ([](float a, float b) { __nv_bfloat162 t = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&t); })(v[4], v[5]);
  o.w = ([](float a, float b) { __nv_bfloat162 t = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&t); })(v[6], v[7]);
  *reinterpret_cast<uint4*>(dst) = o;
}

// First weight row of each half of tile column `tn` (a plain tile of 128 columns has only the first). A SwiGLU
// tile is BN / 2 gate rows and the matching up rows.
template <int BN>
__device__ __forceinline__ void t5_tile_rows(const T5Args& a, int tn, int& row_lo, int& row_hi) {
  if (a.mode == T5_SWIGLU) {
    row_lo = tn * (BN / 2);              // gate rows
    row_hi = a.inter + tn * (BN / 2);    // the matching up rows
  } else {
    row_lo = tn * BN;
    row_hi = row_lo + 128;
  }
}

// Tile number -> (row tile of tokens, tile column of weights, first and end block of its K range).
struct T5Tile {
  int tm, tn, kb0, kb1;
};
__device__ __forceinline__ T5Tile t5_tile(const T5Args& a, int tile, int n_kb) {
  T5Tile t;
  t.tm = tile % a.n_tiles_m;
  const int rest = tile / a.n_tiles_m;
  const int ks = rest % a.n_splits;
  t.tn = rest / a.n_splits;
  t.kb0 = ks * a.kb_per_split;
  t.kb1 = a.n_splits > 1 ? min(n_kb, t.kb0 + a.kb_per_split) : n_kb;
  return t;
}

// 16 bytes of float32 added to memory in one instruction.
__device__ __forceinline__ void t5_red_add4(float* dst, const float* v) {
  asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v[0]), "f"(v[1]), "f"(v[2]),
               "f"(v[3]) : "memory");
}

template <int BN>
__global__ void __launch_bounds__(kT5Threads, 1) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                     const __grid_constant__ CUtensorMap map_w,
                                                                     const T5Args a) {
  constexpr int kT5BN = BN, kT5Stages = t5_stages<BN>(), kT5BBytes = t5_b_bytes<BN>(), kT5StageBytes = t5_stage_bytes<BN>();
  extern __shared__ __align__(1024) unsigned char t5_smem_raw[];
  // The dynamic region is used from the next 1024-byte boundary (the swizzle pattern repeats every 1024 B).
  const uint32_t ring = (t5_smem(t5_smem_raw) + 1023u) & ~1023u;
  __shared__ __align__(8) uint64_t bars[2 * kT5Stages + 4];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  const uint32_t bar0 = t5_smem(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kT5Stages + s); };
  auto tfull_bar = [&](int acc) { return bar0 + 8u * (2 * kT5Stages + acc); };
  auto tempty_bar = [&](int acc) { return bar0 + 8u * (2 * kT5Stages + 2 + acc); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < kT5Stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int acc = 0; acc < 2; ++acc) {
      mbar_init(tfull_bar(acc), 1);
      mbar_init(tempty_bar(acc), 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(t5_smem(&s_tmem_base)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  t5_fence_before();
  __syncthreads();
  t5_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  // (Launched with programmatic dependent launch where it follows a kernel of this library in a decode step: what
  // stands above depends on no earlier kernel, and neither do the weights: the producer asks for its first tile's
  // weight blocks before it waits for the kernel in front. Everything else may read what that kernel wrote.)
  pdl_launch_dependents();
  const bool producer = warp == 0 && lane == 0;
  if (!producer) pdl_wait();

  const int n_tiles = a.n_tiles_m * a.n_tiles_n * a.n_splits;
  const int n_kb = (a.K + kT5BK - 1) / kT5BK;

  if (producer) {
    // ---- TMA producer ----
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int pre = 0;                               // k-blocks of the first tile asked for ahead of the wait
    const bool two_boxes = BN == 256 || a.mode == T5_SWIGLU;   // the weight tile is two boxes of BN / 2 rows
    if ((int)blockIdx.x < n_tiles) {
      const T5Tile tl = t5_tile(a, blockIdx.x, n_kb);
      int row_lo, row_hi;
      t5_tile_rows<BN>(a, tl.tn, row_lo, row_hi);
      pre = min(tl.kb1 - tl.kb0, kT5Stages);
      for (int i = 0; i < pre; ++i) {          // (every stage is free at the start)
        const uint32_t dst = ring + i * kT5StageBytes;
        mbar_expect_tx(full_bar(i), kT5StageBytes);
        tma_load_2d(dst + kT5ABytes, &map_w, (tl.kb0 + i) * kT5BK, row_lo, full_bar(i));
        if (two_boxes) tma_load_2d(dst + kT5ABytes + kT5BBytes / 2, &map_w, (tl.kb0 + i) * kT5BK, row_hi, full_bar(i));
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i)
        tma_load_2d(ring + i * kT5StageBytes, &map_x, (tl.kb0 + i) * kT5BK, tl.tm * kT5BM, full_bar(i));
      stage = pre % kT5Stages;
      if (pre == kT5Stages) phase ^= 1u;
    } else {
      pdl_wait();
    }
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const T5Tile tl = t5_tile(a, tile, n_kb);
      const int tn = tl.tn, tm = tl.tm;
      int row_lo, row_hi;
      t5_tile_rows<BN>(a, tn, row_lo, row_hi);
      for (int kb = tl.kb0 + (tile == (int)blockIdx.x ? pre : 0); kb < tl.kb1 && ok; ++kb) {
        ok = mbar_wait(empty_bar(stage), phase ^ 1u, &s_abort, a.error, 1);
        if (!ok) break;
        const uint32_t dst = ring + stage * kT5StageBytes;
        mbar_expect_tx(full_bar(stage), kT5StageBytes);
        tma_load_2d(dst, &map_x, kb * kT5BK, tm * kT5BM, full_bar(stage));
        tma_load_2d(dst + kT5ABytes, &map_w, kb * kT5BK, row_lo, full_bar(stage));
        if (two_boxes) tma_load_2d(dst + kT5ABytes + kT5BBytes / 2, &map_w, kb * kT5BK, row_hi, full_bar(stage));
        if (++stage == kT5Stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer ----
    // Instruction descriptor: D float32, A and B bfloat16, both K-major, N = BN, M = 128.
    constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kT5BN >> 3) << 17) |
                               ((uint32_t)(kT5BM >> 4) << 24);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, &s_abort, a.error, 2);
      if (!ok) break;
      t5_fence_after();
      const uint32_t d_tmem = tmem_base + acc * kT5BN;
      const T5Tile tl = t5_tile(a, tile, n_kb);
      for (int kb = tl.kb0; kb < tl.kb1 && ok; ++kb) {
        ok = mbar_wait(full_bar(stage), phase, &s_abort, a.error, 3);
        if (!ok) break;
        t5_fence_after();
        const uint32_t sa = ring + stage * kT5StageBytes, sb = sa + kT5ABytes;
#pragma unroll
        for (int k = 0; k < kT5BK / 16; ++k)
          t5_mma(d_tmem, t5_desc(sa + k * 32), t5_desc(sb + k * 32), idesc, (kb != tl.kb0 || k != 0) ? 1u : 0u);
        t5_commit(empty_bar(stage));                   // the stage is free once these products are done
        if (++stage == kT5Stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) t5_commit(tfull_bar(acc));               // the accumulator is complete
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  } else if (warp >= 4) {
    // ---- epilogue: warp w reads tensor-memory lanes 32 * (w % 4) .. + 31 ----
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const T5Tile tl = t5_tile(a, tile, n_kb);
      const int tn = tl.tn, tm = tl.tm;
      ok = mbar_wait(tfull_bar(acc), acc_phase, &s_abort, a.error, 4);
      if (!ok) break;
      t5_fence_after();
      const int t = tm * kT5BM + quarter * 32 + lane;           // this thread's token row
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kT5BN;
      const bool row_ok = t < a.T;
      if (a.mode == T5_STORE) {
#pragma unroll 1
        for (int c = 0; c < kT5BN; c += 32) {
          float v[32];
          t5_ld32(taddr + c, v);
          t5_ld_wait();
          const int n = tn * kT5BN + c;
          if (row_ok && n < a.N) {
            __nv_bfloat16* dst = a.out + (size_t)t * a.ldo + n;
            if (n + 32 <= a.N) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) store8_bf16(dst + j, v + j);
            } else {
              for (int j = 0; j < 32 && n + j < a.N; ++j) dst[j] = __float2bfloat16_rn(v[j]);
            }
          }
        }
      } else if (a.mode == T5_ADD_F32) {
        // One piece of the K range: its sums are added into the 32-bit output (the residual stream), 16 bytes an
        // instruction. (N is a multiple of 4 and the rows are 16-byte aligned: the launcher checks.)
#pragma unroll 1
        for (int c = 0; c < kT5BN; c += 32) {
          float v[32];
          t5_ld32(taddr + c, v);
          t5_ld_wait();
          const int n = tn * kT5BN + c;
          if (row_ok && n < a.N) {
            float* dst = a.out_f32 + (size_t)t * a.ldo + n;
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              if (n + j < a.N) t5_red_add4(dst + j, v + j);
          }
        }
      } else if (a.mode == T5_SWIGLU) {
        constexpr int HALF = BN / 2;       // gate columns, then as many up columns
#pragma unroll 1
        for (int c = 0; c < HALF; c += 32) {
          float g[32], u[32];
          t5_ld32(taddr + c, g);
          t5_ld32(taddr + HALF + c, u);
          t5_ld_wait();
          const int n = tn * HALF + c;
          if (row_ok && n < a.inter) {
#pragma unroll
            for (int j = 0; j < 32; ++j) g[j] = g[j] / (1.0f + expf(-g[j])) * u[j];
            __nv_bfloat16* dst = a.out + (size_t)t * a.ldo + n;
            if (n + 32 <= a.inter) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) store8_bf16(dst + j, g + j);
            } else {
              for (int j = 0; j < 32 && n + j < a.inter; ++j) dst[j] = __float2bfloat16_rn(g[j]);
            }
          }
        }
      } else {
        // QKV: the tile's 256 columns are whole heads (D divides 256); a rotation pair is i and i + D/2.
        const int half = a.D >> 1;
        int pos = 0, slot = -1;
        if (row_ok) {
          pos = a.positions[t];
          if (pos < 0 || pos >= a.n_pos) {                 // never read outside the tables; tell the host
            if (a.error) atomicCAS(a.error, 0, 31);
            pos = pos < 0 ? 0 : a.n_pos - 1;
          }
          slot = a.slot_map ? a.slot_map[t] : -1;
        }
#pragma unroll 1
        for (int hc = 0; hc < kT5BN; hc += a.D) {
          const int head = (tn * kT5BN + hc) / a.D;
          const bool head_ok = head < a.nh + 2 * a.nkv;
#pragma unroll 1
          for (int i0 = 0; i0 < half; i0 += 32) {
            float x1[32], x2[32];
            t5_ld32(taddr + hc + i0, x1);
            t5_ld32(taddr + hc + half + i0, x2);
            t5_ld_wait();
            if (!(row_ok && head_ok)) continue;
            const int c0 = head * a.D + i0, c1 = c0 + half;
            if (a.bias) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                x1[j] += a.bias[c0 + j];
                x2[j] += a.bias[c1 + j];
              }
            }
            if (head < a.nh + a.nkv) {
              const float* cs = a.cos_t + (size_t)pos * half + i0;
              const float* sn = a.sin_t + (size_t)pos * half + i0;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float c = cs[j], s = sn[j];
                const float o1 = __fadd_rn(__fmul_rn(x1[j], c), __fmul_rn(-x2[j], s));
                const float o2 = __fadd_rn(__fmul_rn(x2[j], c), __fmul_rn(x1[j], s));
                x1[j] = o1;
                x2[j] = o2;
              }
            }
            __nv_bfloat16* dst = nullptr;
            if (head < a.nh) {
              dst = a.q_out + ((size_t)t * a.nh + head) * a.D;
            } else if (slot >= 0) {
              const bool is_k = head < a.nh + a.nkv;
              dst = (is_k ? a.kcache : a.vcache) + ((size_t)slot * a.nkv + (is_k ? head - a.nh : head - a.nh - a.nkv)) * a.D;
            }
            if (dst) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                store8_bf16(dst + i0 + j, x1 + j);
                store8_bf16(dst + half + i0 + j, x2 + j);
              }
            }
          }
        }
      }
      // This warp has read everything it needs from the accumulator.
      t5_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // Teardown: every role has left its loop (normally, or through a bounded wait).
  t5_fence_before();
  __syncthreads();
  if (warp == 2) {
    t5_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
  }
}

// --- host -----------------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// A [rows, K] bfloat16 row-major matrix viewed through boxes of 128 (or box_rows) rows x 64 columns, 128-byte swizzle;
// parts of a box outside the matrix read as zero.
static bool make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long row_stride_elems,
                     int box_rows = 128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_stride_elems * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kT5BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1u, 1u};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int t5_sm_count() {
  static int n_sm = 0;
  if (!n_sm) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
  }
  return n_sm;
}

template <int BN>
static int t5_launch(T5Args a, const void* x, int ldx, const void* w, cudaStream_t stream) {
  if (a.T <= 0) return 0;
  if (a.K % 8 || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return TM_ERR_UNSUPPORTED_SHAPE;     // TMA wants 16-byte aligned rows
  if (!a.error) return TM_ERR_SCRATCH_TOO_SMALL;
  CUtensorMap map_x, map_w;
  if (!make_map(&map_x, x, a.T, a.K, ldx) || !make_map(&map_w, w, a.N, a.K, a.K, BN == 64 ? 32 : 128)) return 90006;
  a.n_tiles_m = (a.T + kT5BM - 1) / kT5BM;
  if (a.n_splits <= 0) {
    a.n_splits = 1;
    a.kb_per_split = (a.K + kT5BK - 1) / kT5BK;
  }
  const int n_sm = t5_sm_count();
  const int smem = t5_stages<BN>() * t5_stage_bytes<BN>() + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int tiles = a.n_tiles_m * a.n_tiles_n * a.n_splits;
  const int grid = tiles < n_sm ? tiles : n_sm;
  if (a.mode == T5_ADD_F32 || a.pdl)      // a decode step's product between kernels of this library
    return launch_pdl(gemm_tcgen05_kernel<BN>, dim3(grid), dim3(kT5Threads), (size_t)smem, stream, map_x, map_w, a);
  gemm_tcgen05_kernel<BN><<<grid, kT5Threads, smem, stream>>>(map_x, map_w, a);
  return launch_status();
}

}  // namespace tmk

// out [T, N] = x [T, K] . w [N, K]^T, all bfloat16. `error` is a device int that must be zero; a block
// whose wait runs out writes a non-zero code there instead of hanging.
extern "C" int tm_tc_linear(const void* x, int ldx, const void* w, void* out, int ldo, int T, int N, int K,
                            int* error, cudaStream_t stream) {
  tmk::T5Args a{};
  a.T = T; a.N = N; a.K = K; a.mode = tmk::T5_STORE;
  a.out = (__nv_bfloat16*)out; a.ldo = ldo; a.error = error;
  if (ldo % 8 || (reinterpret_cast<uintptr_t>(out) & 15)) return TM_ERR_UNSUPPORTED_SHAPE;
  // Tiles of 128 columns while tiles of 256 would not fill the chip once (a narrow projection such as o_proj).
  if (((T + tmk::kT5BM - 1) / tmk::kT5BM) * ((N + 255) / 256) < tmk::t5_sm_count()) {
    a.n_tiles_n = (N + 127) / 128;
    return tmk::t5_launch<128>(a, x, ldx, w, stream);
  }
  a.n_tiles_n = (N + 255) / 256;
  return tmk::t5_launch<256>(a, x, ldx, w, stream);
}

// out [T, N] (float32, row stride ldo) += x [T, K] . w [N, K]^T: a projection added into the 32-bit residual stream
// (src/infer/model/qwen2.py:20-22), for steps of a few dozen tokens, where a product is one pass over the weights
// and has too few tiles of 128 columns to fill the chip: the K range is cut so that about one (tile, piece) falls
// to every multiprocessor, and every piece adds its sums with vector atomics (so the order of the sum, and with
// it the last bits, varies from run to run). N a multiple of 4; out 16-byte aligned, ldo a multiple of 4.
extern "C" int tm_tc_linear_add_f32(const void* x, int ldx, const void* w, float* out, int ldo, int T, int N, int K,
                                    int* error, cudaStream_t stream) {
  tmk::T5Args a{};
  a.T = T; a.N = N; a.K = K; a.mode = tmk::T5_ADD_F32;
  a.out_f32 = out; a.ldo = ldo; a.error = error;
  if (N % 4 || ldo % 4 || (reinterpret_cast<uintptr_t>(out) & 15)) return TM_ERR_UNSUPPORTED_SHAPE;
  a.n_tiles_n = (N + 127) / 128;
  const int tiles = ((T + tmk::kT5BM - 1) / tmk::kT5BM) * a.n_tiles_n;
  const int n_kb = (K + tmk::kT5BK - 1) / tmk::kT5BK;
  int splits = tmk::t5_sm_count() / (tiles > 0 ? tiles : 1);
  splits = splits < 1 ? 1 : (splits > n_kb ? n_kb : splits);
  a.kb_per_split = (n_kb + splits - 1) / splits;
  a.n_splits = (n_kb + a.kb_per_split - 1) / a.kb_per_split;
  return tmk::t5_launch<128>(a, x, ldx, w, stream);
}

// out [T, I] = silu(x . gate^T) * (x . up^T); w [2 I, K] with the gate rows first; I a multiple of 8.
extern "C" int tm_tc_gate_up_swiglu(const void* x, int ldx, const void* w, void* out, int ldo, int T, int K,
                                    int inter, int* error, cudaStream_t stream) {
  tmk::T5Args a{};
  a.T = T; a.N = 2 * inter; a.K = K; a.mode = tmk::T5_SWIGLU; a.inter = inter;
  a.out = (__nv_bfloat16*)out; a.ldo = ldo; a.error = error;
  if (ldo % 8 || inter % 8 || (reinterpret_cast<uintptr_t>(out) & 15)) return TM_ERR_UNSUPPORTED_SHAPE;
  if (T <= tmk::kT5BM) {
    // One row tile of tokens (a decode step): tiles of 32 gate and 32 up rows, so that there is one for every
    // multiprocessor (152 for 4,864 rows), launched with programmatic dependent launch.
    a.n_tiles_n = (inter + 31) / 32;
    a.pdl = 1;
    return tmk::t5_launch<64>(a, x, ldx, w, stream);
  }
  a.n_tiles_n = (inter + 127) / 128;
  return tmk::t5_launch<256>(a, x, ldx, w, stream);
}

// Fused q/k/v projection with bias, rotate-half position encoding and cache write (see rope_cache.cu for the
// formulas). Head sizes 64, 128 and 256 (a 256-column tile must hold whole heads; half a head in steps of 32).
extern "C" int tm_tc_qkv_rope_write(const void* x, int ldx, const void* w, const float* bias, const int* positions,
                                    const float* cos_t, const float* sin_t, const int* slot_map, void* q_out,
                                    void* kcache, void* vcache, int T, int K, int nh, int nkv, int D, int n_pos,
                                    int* error, cudaStream_t stream) {
  if (D != 64 && D != 128 && D != 256) return TM_ERR_UNSUPPORTED_SHAPE;
  tmk::T5Args a{};
  a.T = T; a.N = (nh + 2 * nkv) * D; a.K = K; a.mode = tmk::T5_QKV;
  a.bias = bias; a.positions = positions; a.cos_t = cos_t; a.sin_t = sin_t; a.slot_map = slot_map;
  a.q_out = (__nv_bfloat16*)q_out; a.kcache = (__nv_bfloat16*)kcache; a.vcache = (__nv_bfloat16*)vcache;
  a.nh = nh; a.nkv = nkv; a.D = D; a.n_pos = n_pos; a.error = error;
  // Tiles of 128 columns (whole heads of 64 or 128) while tiles of 256 would not fill the chip once.
  const int tiles_m = (T + tmk::kT5BM - 1) / tmk::kT5BM;
  if (D <= 128 && tiles_m * ((a.N + 255) / 256) < tmk::t5_sm_count()) {
    a.n_tiles_n = (a.N + 127) / 128;
    return tmk::t5_launch<128>(a, x, ldx, w, stream);
  }
  a.n_tiles_n = (a.N + 255) / 256;
  return tmk::t5_launch<256>(a, x, ldx, w, stream);
}
