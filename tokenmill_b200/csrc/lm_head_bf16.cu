// The output matrix product of a decode step: logits[T, N] = x[T, K] . w[N, K]^T for T <= 16 tokens and a
// vocabulary-sized N (src/infer/model/qwen2.py:50-52: the output matrix, tied to the embedding or its own),
// bfloat16 in, float32 accumulation and output.
//
// The product reads every weight once and does next to no arithmetic, so it runs at the speed of the memory:
// 272 MB for a vocabulary of 151,936 by 896. Measured on a B200: 52 us with a clean L2 and 64 us behind a
// kernel that left the L2 full of written lines, against 50 and 64 us for the library's kernel: both sit at
// the rate at which the memory can be read (5.2 to 5.4 TB/s), so the engine keeps the library product unless
// asked otherwise, and saves the packed copy. This kernel streams the weights through a ring of shared-memory stages with bulk asynchronous copies
// that complete on mbarriers, several stages ahead of the arithmetic, from the PACKED copy of the matrix
// ([N/8 row groups][K/32 chunks][8 rows][4 pieces][8 elements]: a stage is one contiguous range, and a
// warp's fragment load from it is 512 contiguous bytes).
//
// One persistent block per SM, 8 warps. A stage holds two row groups (16 vocabulary rows). Warp w works on row
// group w / 4 and on the quarter w % 4 of the K range, with the tokens' activations for that quarter in its
// registers for the whole kernel (tokens are the M side of mma.m16n8k16, the 8 rows of the group its N side;
// the k index inside a 32-element chunk is permuted the same way on both sides, so that a lane's 16-byte
// weight load is two instructions' worth of B fragments). The four quarters of a row group meet in shared
// memory in a fixed order, and 256 threads write the 2 x 16 x 8 results of the stage.
//
// The stages of the ring are filled before the kernel waits for the kernel in front of it on the stream
// (programmatic dependent launch): the weights depend on nothing. Every mbarrier wait is bounded; a block whose
// wait runs out raises the error word and leaves.
#include "tcgen05_util.cuh"
#include "mma_util.cuh"

namespace tmk {

constexpr int kLhThreads = 256;
constexpr int kLhMaxChunksPerWarp = 8;      // K <= 4 * 8 * 32 = 1024

struct LmHeadArgs {
  const __nv_bfloat16* x;      // [T, K]
  const __nv_bfloat16* w;      // packed
  float* out;                  // [T, N]
  int T, N, K;
  int chunks;                  // K / 32 rounded up
  int n_stages_total;          // row-group pairs
  int ring;                    // stages in shared memory
  int n_slices;                // cuts of the K range; a block works on one of them (blockIdx.x % n_slices)
  int slice_chunks;            // chunks of a slice (the last may have fewer)
  long long slice_stride;      // floats between two slices' outputs (T * N), 0 with one slice
  int* error;
  // Arg-max in the epilogue (one slice only; all null when not asked for): every block keeps, per token, the
  // largest of the logits it computed (the lowest index on ties) and writes it to best_val / best_idx
  // [grid, 16]; the block that finishes last (arrival counter `done`, zero between launches) picks each
  // token's winner over the blocks in index order and writes argmax_out [T].
  int* argmax_out;
  float* best_val;
  int* best_idx;
  int* done;
};

// (value, index) pairs: the larger value wins, the lower index on equal values (torch.argmax's rule).
__device__ __forceinline__ void lh_better(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) {
    v = ov;
    i = oi;
  }
}

template <int CPW>   // chunks of 32 k per warp
__global__ void __launch_bounds__(kLhThreads, 1) lm_head_kernel(const LmHeadArgs a) {
  extern __shared__ __align__(1024) unsigned char lh_smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int group = warp >> 2, quarter = warp & 3;
  // A wide K range is cut into slices of at most 1024 columns (what a warp's registers hold of the
  // activations); a block keeps one slice for all its row groups and writes that slice's partial sums.
  const int slice = (int)blockIdx.x % a.n_slices;
  const int my_chunks = min(a.slice_chunks, a.chunks - slice * a.slice_chunks);
  const int pair0 = (int)blockIdx.x / a.n_slices, pair_step = (int)gridDim.x / a.n_slices;
  const uint32_t group_bytes = (uint32_t)a.slice_chunks * 512u, stage_bytes = 2u * group_bytes;
  const uint32_t base = t5_smem(lh_smem);
  // shared memory: ring stages, then the partial sums (2 buffers x 8 warps x 32 lanes x 4 floats), then barriers
  float* red = reinterpret_cast<float*>(lh_smem + (size_t)a.ring * stage_bytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + 2 * 8 * 128);
  volatile int* s_abort = reinterpret_cast<volatile int*>(bars + a.ring);
  const int n_groups = (a.N + 7) >> 3;

  if (tid == 0) {
    *s_abort = 0;
    for (int s = 0; s < a.ring; ++s) mbar_init(t5_smem(&bars[s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // this block's stages: row-group pairs pair0, pair0 + pair_step, ... (all of its own slice)
  const int my_stages = a.n_stages_total > pair0 ? (a.n_stages_total - 1 - pair0) / pair_step + 1 : 0;
  auto issue = [&](int it) {                 // one thread: stage `it` of this block into ring slot it % ring
    const int st = pair0 + it * pair_step;
    const int groups_here = min(2, n_groups - 2 * st);
    const uint32_t bytes = (uint32_t)my_chunks * 512u;
    const uint32_t bar = t5_smem(&bars[it % a.ring]);
    mbar_expect_tx(bar, (uint32_t)groups_here * bytes);
    for (int gi = 0; gi < groups_here; ++gi)       // a group's chunks of this slice are one contiguous range
      bulk_load(base + (uint32_t)(it % a.ring) * stage_bytes + (uint32_t)gi * group_bytes,
                reinterpret_cast<const unsigned char*>(a.w) +
                    ((size_t)(2 * st + gi) * a.chunks + (size_t)slice * a.slice_chunks) * 512, bytes, bar);
  };
  if (tid == 0)
    for (int it = 0; it < a.ring && it < my_stages; ++it) issue(it);

  pdl_launch_dependents();
  pdl_wait();                                // the activations come from the kernel before

  // The tokens' activations for this warp's quarter of K: chunk c of the quarter, tokens g and g + 8, columns
  // 8 t .. 8 t + 7 of the chunk.
  uint32_t xlo[CPW][4], xhi[CPW][4];
#pragma unroll
  for (int c = 0; c < CPW; ++c) {
    const int k = ((slice * a.slice_chunks + quarter * CPW + c) * 32) + 8 * t;
    uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
    if (quarter * CPW + c < my_chunks && k < a.K) {      // K is a multiple of 8: a piece is whole or absent
      if (g < a.T) lo = *reinterpret_cast<const uint4*>(a.x + (size_t)g * a.K + k);
      if (g + 8 < a.T) hi = *reinterpret_cast<const uint4*>(a.x + (size_t)(g + 8) * a.K + k);
    }
    xlo[c][0] = lo.x; xlo[c][1] = lo.y; xlo[c][2] = lo.z; xlo[c][3] = lo.w;
    xhi[c][0] = hi.x; xhi[c][1] = hi.y; xhi[c][2] = hi.z; xhi[c][3] = hi.w;
  }

  float best = -INFINITY;                    // this thread's largest logit so far (its token: (tid >> 3) & 15)
  int best_n = 0x7fffffff;
  int it = 0;
  for (; it < my_stages; ++it) {
    const int slot = it % a.ring;
    // (A wait that runs out sets the block's abort flag; the block leaves together after the barrier below.)
    const bool ok = mbar_wait(t5_smem(&bars[slot]), (uint32_t)(it / a.ring) & 1u, s_abort, a.error, 21);
    float c4[4] = {0.f, 0.f, 0.f, 0.f};
    if (ok) {
      const uint32_t wbase = base + (uint32_t)slot * stage_bytes + (uint32_t)group * group_bytes + (uint32_t)lane * 16u;
#pragma unroll
      for (int c = 0; c < CPW; ++c) {
        const int chunk = quarter * CPW + c;
        if (chunk < my_chunks) {
          uint32_t w0, w1, w2, w3;
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3) : "r"(wbase + (uint32_t)chunk * 512u));
          const uint32_t a0[4] = {xlo[c][0], xhi[c][0], xlo[c][1], xhi[c][1]};
          const uint32_t a1[4] = {xlo[c][2], xhi[c][2], xlo[c][3], xhi[c][3]};
          mma_bf16_16816(c4, a0, w0, w1);
          mma_bf16_16816(c4, a1, w2, w3);
        }
      }
    }
    float* mine = red + ((it & 1) * 8 + warp) * 128;
    *reinterpret_cast<float4*>(mine + lane * 4) = make_float4(c4[0], c4[1], c4[2], c4[3]);
    __syncthreads();                         // the stage has been read by everyone; the partial sums are visible
    if (*s_abort) break;                     // the same for every thread: the flag was set before the barrier
    if (tid == 0 && it + a.ring < my_stages) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the reads of the slot come before its refill
      issue(it + a.ring);
    }
    // thread -> (row group of the stage, token, row of the group); the four quarters of K in order
    const int grp = tid >> 7, tok = (tid >> 3) & 15, col = tid & 7;
    const int src_lane = (tok & 7) * 4 + (col >> 1), src_reg = (tok >> 3) * 2 + (col & 1);
    const float* p = red + ((it & 1) * 8 + grp * 4) * 128 + src_lane * 4 + src_reg;
    const float sum = ((p[0] + p[128]) + p[256]) + p[384];
    const int st = pair0 + it * pair_step;
    const int n = (2 * st + grp) * 8 + col;
    if (tok < a.T && n < a.N) {
      if (a.out) a.out[(size_t)slice * a.slice_stride + (size_t)tok * a.N + n] = sum;
      if (sum > best) {                      // (n grows from stage to stage: the first of equal values stays)
        best = sum;
        best_n = n;
      }
    }
  }
  if (a.argmax_out && it == my_stages) {
    // A token's 16 threads: 8 neighbouring lanes (the rows of a group) in each of two warps (the two groups).
    __shared__ float s_val[2][16];
    __shared__ int s_idx[2][16];
    __shared__ int s_last;
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_n, o);
      lh_better(best, best_n, ov, oi);
    }
    __syncthreads();
    if ((tid & 7) == 0) {
      s_val[tid >> 7][(tid >> 3) & 15] = best;
      s_idx[tid >> 7][(tid >> 3) & 15] = best_n;
    }
    __syncthreads();
    if (tid < 16) {
      float v = s_val[0][tid];
      int i = s_idx[0][tid];
      lh_better(v, i, s_val[1][tid], s_idx[1][tid]);
      a.best_val[(size_t)blockIdx.x * 16 + tid] = v;
      a.best_idx[(size_t)blockIdx.x * 16 + tid] = i;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(a.done, 1) == (int)gridDim.x - 1;
    __syncthreads();
    if (s_last) {
      __threadfence();
      // 16 threads per token, each over every 16th block, then the lowest index among equal values again
      // (the rule is symmetric, so the order in which pairs meet does not matter).
      const int tok = tid >> 4, part = tid & 15;
      float v = -INFINITY;
      int i = 0x7fffffff;
      for (int b = part; b < (int)gridDim.x; b += 16)
        lh_better(v, i, __ldcg(a.best_val + (size_t)b * 16 + tok), __ldcg(a.best_idx + (size_t)b * 16 + tok));
#pragma unroll
      for (int o = 1; o < 16; o <<= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        lh_better(v, i, ov, oi);
      }
      if (part == 0 && tok < a.T) a.argmax_out[tok] = i;
      if (tid == 0) *a.done = 0;
    }
  }
  // After an abort: the copies still on their way into this block's shared memory are waited for (bounded)
  // before the block gives the memory up.
  if (it < my_stages && tid == 0) {
    for (int j = it + 1; j < my_stages && j < it + a.ring; ++j) {
      const uint32_t bar = t5_smem(&bars[j % a.ring]);
      for (uint32_t spin = 0; spin < (1u << 20) && !mbar_try(bar, (uint32_t)(j / a.ring) & 1u); ++spin) __nanosleep(64);
    }
  }
}

}  // namespace tmk

// How many slices of the K range tm_stream_linear_bf16 cuts a product of K columns into (each at most 1024
// columns, all but the last equally long): the caller sizes the output by it.
extern "C" int tm_stream_linear_slices(int K) {
  const int chunks = (K + 31) / 32;
  return (chunks + 31) / 32;
}

// x [T, K] bfloat16 (T <= 16, K a multiple of 8), w_packed the packed copy of w [N, K] (rows padded to a
// multiple of 8, K to a multiple of 32), out [n_slices, T, N] float32 with n_slices = tm_stream_linear_slices(K):
// slice s holds the sums over its part of the K range (the caller, or the norm kernel that follows, adds the
// slices in index order). `error`: a device int that must be zero; a block whose wait runs out writes 21 there
// instead of hanging.
static int lh_launch(const void* x, const void* w_packed, float* out, int T, int N, int K, int* error, int* argmax_out,
                     float* best_val, int* best_idx, int* done, cudaStream_t stream);

extern "C" int tm_stream_linear_bf16(const void* x, const void* w_packed, float* out, int T, int N, int K, int* error,
                                     cudaStream_t stream) {
  if (!out) return TM_ERR_UNSUPPORTED_SHAPE;
  return lh_launch(x, w_packed, out, T, N, K, error, nullptr, nullptr, nullptr, nullptr, stream);
}

static int lh_launch(const void* x, const void* w_packed, float* out, int T, int N, int K, int* error, int* argmax_out,
                     float* best_val, int* best_idx, int* done, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (T > 16 || K <= 0 || K % 8 || !error) return TM_ERR_UNSUPPORTED_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w_packed)) & 15) return TM_ERR_UNSUPPORTED_SHAPE;
  static int n_sm = 0;
  if (!n_sm) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
  }
  const int chunks = (K + 31) / 32;
  const int n_slices = tm_stream_linear_slices(K);
  if (n_slices > n_sm) return TM_ERR_UNSUPPORTED_SHAPE;
  const int slice_chunks = (chunks + n_slices - 1) / n_slices;
  const int cpw = (slice_chunks + 3) / 4;
  if (cpw > tmk::kLhMaxChunksPerWarp || (long long)slice_chunks * (n_slices - 1) >= chunks) return TM_ERR_UNSUPPORTED_SHAPE;
  tmk::LmHeadArgs a{};
  a.x = (const __nv_bfloat16*)x; a.w = (const __nv_bfloat16*)w_packed; a.out = out;
  a.T = T; a.N = N; a.K = K; a.chunks = chunks; a.error = error;
  a.argmax_out = argmax_out; a.best_val = best_val; a.best_idx = best_idx; a.done = done;
  if (argmax_out && (n_slices != 1 || !best_val || !best_idx || !done)) return TM_ERR_UNSUPPORTED_SHAPE;
  a.n_slices = n_slices; a.slice_chunks = slice_chunks; a.slice_stride = n_slices > 1 ? (long long)T * N : 0;
  const int n_groups = (N + 7) / 8;
  a.n_stages_total = (n_groups + 1) / 2;
  const size_t stage_bytes = (size_t)2 * slice_chunks * 512;
  const size_t fixed = 2 * 8 * 128 * sizeof(float) + 64 * sizeof(uint64_t) + 64;
  int ring = (int)((200 * 1024 - fixed) / stage_bytes);
  if (ring > 32) ring = 32;
  if (ring < 2) return TM_ERR_UNSUPPORTED_SHAPE;
  a.ring = ring;
  const size_t smem = (size_t)ring * stage_bytes + fixed;
  int per_slice = n_sm / n_slices;                       // blocks per slice: the grid is a multiple of n_slices
  if (per_slice > a.n_stages_total) per_slice = a.n_stages_total;
  const int grid = per_slice * n_slices;
#define LH_CASE(C)                                                                                               \
  {                                                                                                              \
    auto kern = tmk::lm_head_kernel<C>;                                                                          \
    static bool set = false;                                                                                     \
    if (!set) {                                                                                                  \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);       \
      if (e != cudaSuccess) return (int)e;                                                                       \
      set = true;                                                                                                \
    }                                                                                                            \
    return tmk::launch_pdl(kern, dim3(grid), dim3(tmk::kLhThreads), smem, stream, a);                            \
  }
  if (cpw <= 1) LH_CASE(1)
  if (cpw <= 2) LH_CASE(2)
  if (cpw <= 4) LH_CASE(4)
  if (cpw <= 7) LH_CASE(7)
  LH_CASE(8)
#undef LH_CASE
}

// The output matrix of a decode step: tm_stream_linear_bf16 for a K of at most 1024 columns (one slice), out [T, N].
extern "C" int tm_lm_head_bf16(const void* x, const void* w_packed, float* out, int T, int N, int K, int* error,
                               cudaStream_t stream) {
  if (K > 1024) return TM_ERR_UNSUPPORTED_SHAPE;
  return tm_stream_linear_bf16(x, w_packed, out, T, N, K, error, stream);
}

// The same product with the arg-max of every token's logits found in the epilogue: tokens [T] int32 receives the
// index of the largest logit (the lowest index on ties), so a greedy decode step neither writes nor re-reads
// [T, N] logits (the reference computes logits.argmax(-1) as a separate pass, src/infer/sampling.py:30-33).
// `logits` may be null (nothing is written) or [T, N] float32. Scratch: best_val, best_idx [148 * 16] (one row per
// block; any number of blocks up to the device's SMs), done: one int that is zero (left zero).
extern "C" int tm_lm_head_argmax_bf16(const void* x, const void* w_packed, float* logits, int* tokens, float* best_val,
                                      int* best_idx, int* done, int T, int N, int K, int* error, cudaStream_t stream) {
  if (K > 1024 || !tokens) return TM_ERR_UNSUPPORTED_SHAPE;
  return lh_launch(x, w_packed, logits, T, N, K, error, tokens, best_val, best_idx, done, stream);
}
