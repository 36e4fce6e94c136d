// Weight-streaming matrix product for decode steps: out[T, N] = x[T, K] . W[N, K]^T with T <= 64
// tokens, bfloat16 operands, float32 accumulation, and the epilogue of whichever projection it is.
//
// At these sizes the product is bound by reading W once from HBM; the tokens are an afterthought.
// So the work is cut along W: a block owns NG groups of 8 weight rows (output features) and, inside
// the block, the K range is cut across the 8 / NG warps of each group. A warp streams its 8 rows
// straight from global memory, 16 bytes per lane (lane = row * 4 + quarter of a 32-wide k chunk), and
// feeds them as the B operand of mma.sync.m16n8k16 against the tokens' activations, which sit in shared
// memory (A operand; the k order inside a chunk is permuted the same way for both operands, which a dot
// product does not mind). The warps' partial sums meet in shared memory and are added in warp order, so
// results do not depend on scheduling. Optionally the K range is also cut across blockIdx.y; then
// 32-bit partial products are written for the following add+norm kernel to sum in index order.
//
// Epilogues (the reference's projections, src/infer/model/layers.py:127-164, qwen2.py:51-52):
//   STORE    out[t, n] (+ bias[n]) in bfloat16 or float32                      (o_proj, output matrix)
//   PARTIAL  partials[y, t, n] in float32                                       (o_proj, down_proj)
//   QKV      + bias, rotate-half position encoding of q and k, q to q_out, k and v to their cache slot
//   SWIGLU   out[t, i] = silu(gate_i) * up_i, gate rows [0, I), up rows [I, 2I) of W
// tcgen05 is not used here on purpose: its smallest tile is 64 weight rows, which would leave most
// SMs without a block for the 896-row projections, and the kernel is bandwidth-bound either way.
#include "common.cuh"

namespace tmk {

constexpr int kSkWarps = 8;
enum : int { SK_STORE = 0, SK_PARTIAL = 1, SK_QKV = 2, SK_SWIGLU = 3 };

struct SkinnyArgs {
  const __nv_bfloat16* x;     // [T, K] row stride ldx
  const __nv_bfloat16* w;     // [N, K]
  int ldx, T, N, K;
  int k_per_block;            // K range of one blockIdx.y (multiple of 32, or K)
  int ng;                     // feature groups (of 8 rows) per block: 1, 2, 4 or 8
  int mode;
  // STORE / PARTIAL / SWIGLU
  void* out;                  // bf16 or f32 [T, ldo]
  int ldo, out_f32;
  const float* bias;          // [N] or null
  float* partials;            // [splits, T, N]
  long long partial_stride;
  // QKV
  const int* positions;
  const float* cos_t;
  const float* sin_t;
  const int* slot_map;
  __nv_bfloat16* q_out;
  __nv_bfloat16* kcache;
  __nv_bfloat16* vcache;
  int nh, nkv, D, n_pos;
  int* error;                 // QKV: set to 31 when a position lies outside the tables (may be null)
  int inter;                  // SWIGLU: I
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void sk_cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void sk_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// First weight row of feature group g of block bx.
__device__ __forceinline__ int sk_group_row(const SkinnyArgs& a, int bx, int g) {
  if (a.mode == SK_QKV) {          // block = (head, 8-wide slice of the first half); group 1 is the rotation partner
    const int per_head = a.D / 16;
    const int head = bx / per_head, i0 = (bx - head * per_head) * 8;
    return head * a.D + i0 + g * (a.D / 2);
  }
  if (a.mode == SK_SWIGLU) return bx * 8 + g * a.inter;   // gate rows, then the matching up rows
  return (bx * a.ng + g) * 8;
}

template <int MT>   // 16-token tiles: T <= 16 * MT
__global__ void __launch_bounds__(kSkWarps * 32) skinny_gemm_kernel(const SkinnyArgs a) {
  extern __shared__ __align__(16) unsigned char sk_smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kc0 = blockIdx.y * a.k_per_block;
  const int kc1 = min(a.K, kc0 + a.k_per_block);
  const int kspan = kc1 - kc0;                         // multiple of 8
  const int kpad = (kspan + 31) / 32 * 32;
  // Row stride of the activations in shared memory: kpad * 2 bytes plus padding to 64 mod 128, which keeps
  // the 16-byte fragment reads of 8 rows x 4 quarters free of bank conflicts.
  const int row_bytes = kpad * 2 + ((64 - (kpad * 2) % 128) + 128) % 128;
  unsigned char* xs = sk_smem;
  float* red = reinterpret_cast<float*>(sk_smem + (size_t)MT * 16 * row_bytes);   // [8 warps][MT*16][8]

  const int kw = kSkWarps / a.ng;                      // warps per feature group
  const int g = warp / kw, kpart = warp - g * kw;
  const int row0 = sk_group_row(a, blockIdx.x, g);
  const int n_chunks = kpad / 32;
  const int per = (n_chunks + kw - 1) / kw;
  const int c_begin = kpart * per, c_end = min(n_chunks, c_begin + per);
  const int wrow = row0 + (lane >> 2);
  const bool row_ok = wrow < a.N && row0 >= 0;
  const __nv_bfloat16* wp = a.w + (size_t)(row_ok ? wrow : 0) * a.K + kc0 + (lane & 3) * 8;

  float acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;

  constexpr int U = 8;                                  // weight chunks in flight per lane
  uint4 wreg[U];
  auto load_w = [&](int c) -> uint4 {
    const int k = c * 32 + (lane & 3) * 8;
    if (row_ok && c < c_end && k < kspan) return ldg_stream(wp + c * 32);
    return make_uint4(0u, 0u, 0u, 0u);
  };
#pragma unroll
  for (int u = 0; u < U; ++u) wreg[u] = load_w(c_begin + u);   // weights depend on no earlier kernel
  pdl_launch_dependents();
  pdl_wait();                                                  // the activations do

  // Stage the activations (rows beyond T and columns beyond the range are zero).
  {
    const int chunks = kpad / 8;
    const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(xs));
    for (int idx = tid; idx < MT * 16 * chunks; idx += kSkWarps * 32) {
      const int r = idx / chunks, c = idx - r * chunks;
      const bool ok = r < a.T && c * 8 < kspan;
      const __nv_bfloat16* src = ok ? a.x + (size_t)r * a.ldx + kc0 + c * 8 : a.x;
      sk_cp_async16(base + r * row_bytes + c * 16, src, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  }

  asm volatile("cp.async.wait_group 0;\n" ::);
  __syncthreads();

  const unsigned char* xrow = xs + (lane >> 2) * row_bytes + (lane & 3) * 16;
  for (int c = c_begin; c < c_end; c += U) {
    uint4 cur[U];
#pragma unroll
    for (int u = 0; u < U; ++u) cur[u] = wreg[u];
#pragma unroll
    for (int u = 0; u < U; ++u) wreg[u] = load_w(c + U + u);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (c + u < c_end) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const uint4 lo = *reinterpret_cast<const uint4*>(xrow + (size_t)(m * 16) * row_bytes + (c + u) * 64);
          const uint4 hi = *reinterpret_cast<const uint4*>(xrow + (size_t)(m * 16 + 8) * row_bytes + (c + u) * 64);
          sk_mma(acc[m], lo.x, hi.x, lo.y, hi.y, cur[u].x, cur[u].y);
          sk_mma(acc[m], lo.z, hi.z, lo.w, hi.w, cur[u].z, cur[u].w);
        }
      }
    }
  }

  // Partial sums meet in shared memory: red[warp][token][feature].
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const int t0 = m * 16 + (lane >> 2), f = (lane & 3) * 2;
    *reinterpret_cast<float2*>(red + ((size_t)warp * MT * 16 + t0) * 8 + f) = make_float2(acc[m][0], acc[m][1]);
    *reinterpret_cast<float2*>(red + ((size_t)warp * MT * 16 + t0 + 8) * 8 + f) = make_float2(acc[m][2], acc[m][3]);
  }
  __syncthreads();
  auto total = [&](int t, int grp, int f) -> float {
    float s = 0.f;
    for (int p = 0; p < kw; ++p) s += red[((size_t)(grp * kw + p) * MT * 16 + t) * 8 + f];
    return s;
  };

  if (a.mode == SK_QKV) {
    const int per_head = a.D / 16, half = a.D / 2;
    const int head = blockIdx.x / per_head, i0 = (blockIdx.x - head * per_head) * 8;
    for (int idx = tid; idx < a.T * 8; idx += kSkWarps * 32) {
      const int t = idx >> 3, j = idx & 7, i = i0 + j;
      const int c0 = head * a.D + i, c1 = c0 + half;
      float x1 = total(t, 0, j), x2 = total(t, 1, j);
      if (a.bias) {
        x1 += a.bias[c0];
        x2 += a.bias[c1];
      }
      float o1 = x1, o2 = x2;
      if (head < a.nh + a.nkv) {
        int pos = a.positions[t];
        if (pos < 0 || pos >= a.n_pos) {                   // never read outside the tables; tell the host
          if (a.error) atomicCAS(a.error, 0, 31);
          pos = pos < 0 ? 0 : a.n_pos - 1;
        }
        const float cs = a.cos_t[(size_t)pos * half + i], sn = a.sin_t[(size_t)pos * half + i];
        o1 = __fadd_rn(__fmul_rn(x1, cs), __fmul_rn(-x2, sn));
        o2 = __fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn));
      }
      if (head < a.nh) {
        __nv_bfloat16* dst = a.q_out + ((size_t)t * a.nh + head) * a.D;
        dst[i] = __float2bfloat16_rn(o1);
        dst[i + half] = __float2bfloat16_rn(o2);
      } else {
        const int slot = a.slot_map ? a.slot_map[t] : -1;
        if (slot >= 0) {
          const bool is_k = head < a.nh + a.nkv;
          const int kh = is_k ? head - a.nh : head - a.nh - a.nkv;
          __nv_bfloat16* dst = (is_k ? a.kcache : a.vcache) + ((size_t)slot * a.nkv + kh) * a.D;
          dst[i] = __float2bfloat16_rn(o1);
          dst[i + half] = __float2bfloat16_rn(o2);
        }
      }
    }
    return;
  }
  if (a.mode == SK_SWIGLU) {
    for (int idx = tid; idx < a.T * 8; idx += kSkWarps * 32) {
      const int t = idx >> 3, j = idx & 7, n = blockIdx.x * 8 + j;
      if (n >= a.inter) continue;
      const float gt = total(t, 0, j), up = total(t, 1, j);
      const float act = gt / (1.0f + expf(-gt));
      reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)t * a.ldo + n] = __float2bfloat16_rn(act * up);
    }
    return;
  }
  const int feats = a.ng * 8;
  for (int idx = tid; idx < a.T * feats; idx += kSkWarps * 32) {
    const int t = idx / feats, fj = idx - t * feats;
    const int grp = fj >> 3, j = fj & 7;
    const int n = (blockIdx.x * a.ng + grp) * 8 + j;
    if (n >= a.N) continue;
    float v = total(t, grp, j);
    if (a.mode == SK_PARTIAL) {
      a.partials[(size_t)blockIdx.y * a.partial_stride + (size_t)t * a.N + n] = v;
    } else {
      if (a.bias) v += a.bias[n];
      if (a.out_f32) reinterpret_cast<float*>(a.out)[(size_t)t * a.ldo + n] = v;
      else reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)t * a.ldo + n] = __float2bfloat16_rn(v);
    }
  }
}

static int sk_launch(const SkinnyArgs& a, int blocks_x, int blocks_y, cudaStream_t stream) {
  if (a.T <= 0 || blocks_x <= 0) return 0;
  if (a.T > 64 || a.K % 8 || a.K <= 0 || (a.ng != 1 && a.ng != 2 && a.ng != 4 && a.ng != 8)) return TM_ERR_UNSUPPORTED_SHAPE;
  if ((reinterpret_cast<uintptr_t>(a.x) & 15) || (reinterpret_cast<uintptr_t>(a.w) & 15) || (a.ldx % 8))
    return TM_ERR_UNSUPPORTED_SHAPE;
  const int mt = a.T <= 16 ? 1 : (a.T <= 32 ? 2 : 4);
  const int kspan = a.k_per_block < a.K ? a.k_per_block : a.K;
  const int kpad = (kspan + 31) / 32 * 32;
  const int row_bytes = kpad * 2 + ((64 - (kpad * 2) % 128) + 128) % 128;
  const size_t smem = (size_t)mt * 16 * row_bytes + (size_t)kSkWarps * mt * 16 * 8 * sizeof(float);
  if (smem > 220 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
  const dim3 grid(blocks_x, blocks_y);
#define SK_CASE(MTV)                                                                                          \
  {                                                                                                           \
    auto kern = skinny_gemm_kernel<MTV>;                                                                      \
    if (smem > 48 * 1024) {                                                                                   \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
      if (e != cudaSuccess) return (int)e;                                                                    \
    }                                                                                                         \
    const int st = launch_pdl(kern, grid, dim3(kSkWarps * 32), smem, stream, a);                              \
    if (st != 0) return st;                                                                                   \
  }
  if (mt == 1) SK_CASE(1) else if (mt == 2) SK_CASE(2) else SK_CASE(4)
#undef SK_CASE
  return launch_status();
}

}  // namespace tmk

// out[T, N] = x . w^T (+ bias); out is bfloat16, or float32 when out_f32 != 0. k_splits > 1 writes
// float32 partial products partials[k_splits, T, N] instead (out unused).
extern "C" int tm_skinny_linear(const void* x, int ldx, const void* w, const float* bias, void* out, int ldo,
                                int out_f32, float* partials, int k_splits, int T, int N, int K, int ng,
                                cudaStream_t stream) {
  tmk::SkinnyArgs a{};
  a.x = (const __nv_bfloat16*)x;
  a.w = (const __nv_bfloat16*)w;
  a.ldx = ldx; a.T = T; a.N = N; a.K = K; a.ng = ng;
  a.out = out; a.ldo = ldo; a.out_f32 = out_f32; a.bias = bias;
  if (k_splits > 1) {
    if (!partials) return TM_ERR_SCRATCH_TOO_SMALL;
    a.mode = tmk::SK_PARTIAL;
    a.k_per_block = ((K + k_splits - 1) / k_splits + 31) / 32 * 32;
    a.partials = partials;
    a.partial_stride = (long long)T * N;
    if ((long long)a.k_per_block * (k_splits - 1) >= K) return TM_ERR_UNSUPPORTED_SHAPE;   // an empty split
  } else {
    a.mode = tmk::SK_STORE;
    a.k_per_block = K;
    k_splits = 1;
  }
  return tmk::sk_launch(a, (N + 8 * ng - 1) / (8 * ng), k_splits, stream);
}

// Fused q/k/v projection: x [T, K] . w [(nh + 2 nkv) D, K]^T + bias, rotate-half position encoding of q and
// k (tables [n_pos, D/2]), q to q_out [T, nh, D], k and v to their slots of the paged caches.
extern "C" int tm_skinny_qkv_rope_write(const void* x, int ldx, const void* w, const float* bias,
                                        const int* positions, const float* cos_t, const float* sin_t,
                                        const int* slot_map, void* q_out, void* kcache, void* vcache, int T, int K,
                                        int nh, int nkv, int D, int n_pos, int* error, cudaStream_t stream) {
  if (D % 16) return TM_ERR_UNSUPPORTED_SHAPE;
  tmk::SkinnyArgs a{};
  a.x = (const __nv_bfloat16*)x;
  a.w = (const __nv_bfloat16*)w;
  a.ldx = ldx; a.T = T; a.N = (nh + 2 * nkv) * D; a.K = K; a.ng = 2; a.mode = tmk::SK_QKV;
  a.k_per_block = K;
  a.bias = bias; a.positions = positions; a.cos_t = cos_t; a.sin_t = sin_t; a.slot_map = slot_map;
  a.q_out = (__nv_bfloat16*)q_out; a.kcache = (__nv_bfloat16*)kcache; a.vcache = (__nv_bfloat16*)vcache;
  a.nh = nh; a.nkv = nkv; a.D = D; a.n_pos = n_pos; a.error = error;
  return tmk::sk_launch(a, (nh + 2 * nkv) * (D / 16), 1, stream);
}

// Fused gate/up projection with SwiGLU: w [2 I, K] (gate rows first); out [T, I] bfloat16.
extern "C" int tm_skinny_gate_up_swiglu(const void* x, int ldx, const void* w, void* out, int ldo, int T, int K,
                                        int inter, cudaStream_t stream) {
  tmk::SkinnyArgs a{};
  a.x = (const __nv_bfloat16*)x;
  a.w = (const __nv_bfloat16*)w;
  a.ldx = ldx; a.T = T; a.N = 2 * inter; a.K = K; a.ng = 2; a.mode = tmk::SK_SWIGLU;
  a.k_per_block = K; a.out = out; a.ldo = ldo; a.inter = inter;
  return tmk::sk_launch(a, (inter + 7) / 8, 1, stream);
}
