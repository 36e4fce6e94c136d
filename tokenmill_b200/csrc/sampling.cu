// Token selection from 32-bit logits: one block per row, and for rows of 8,192 logits and more a cluster of eight
// blocks per row (sample_cluster_kernel, at the end of this file).
//
// Greedy: the index of the largest logit, the lowest index on ties (torch.argmax's rule, which the
// reference uses: src/infer/sampling.py:30-33).
// Random rows (src/infer/sampling.py:34-45): z = logits / temperature; optional top-k (keep the k
// largest) and top-p (after top-k, drop a token once the probability mass of the tokens ranked before
// it exceeds top_p; the best token always stays); softmax over what is kept; one draw. The draw is an
// inverse-CDF walk over the vocabulary in index order with a uniform number u in [0, 1) the caller
// supplies: the token is the first index whose running sum of kept weights exceeds u * total. The
// reference draws with torch.multinomial from a per-request generator instead; the distribution is
// the same, the stream of numbers is this engine's own. Where the reference sorts, this kernel
// finds the two cut values by bisection on the float bit pattern, so tokens tied exactly at a cut
// are all kept. The bisections run over the few thousand tokens next to the row's maximum, copied to
// shared memory, whenever the cuts lie among them (sample_from_candidates: 0.12 to 0.15 ms a step at a
// vocabulary of 152k with one block per row, 0.03 to 0.05 ms with a cluster), and over the whole row otherwise
// (1 to 1.7 ms with one block, 0.12 ms with a cluster, which keeps the row in shared memory).
#include "common.cuh"

namespace tmk {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ unsigned int float_order_bits(float f) {
  const unsigned int b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);  // monotone: a < b  <=>  bits(a) < bits(b)
}
__device__ __forceinline__ float order_bits_float(unsigned int u) {
  const unsigned int b = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
  return __uint_as_float(b);
}

__global__ void __launch_bounds__(kSampleThreads) argmax_kernel(const float* __restrict__ logits, int V,
                                                               long long row_stride, int* __restrict__ out) {
  __shared__ float sval[32];
  __shared__ int sidx[32];
  const float* row = logits + (size_t)blockIdx.x * row_stride;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sval[warp] = best;
    sidx[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sval[lane] : -INFINITY;
    bi = lane < nw ? sidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

// Two-stage arg-max for wide vocabularies: blockIdx.y takes one chunk of the row and leaves its best
// (value, lowest index); the final kernel reduces the chunks. One block per row would read 600 KB alone.
constexpr int kArgmaxChunk = 4096;

__global__ void __launch_bounds__(256) argmax_chunk_kernel(const float* __restrict__ logits, int V,
                                                          long long row_stride, float* __restrict__ cval,
                                                          int* __restrict__ cidx, int n_chunks) {
  __shared__ float sval[8];
  __shared__ int sidx[8];
  const float* row = logits + (size_t)blockIdx.x * row_stride;
  const int begin = blockIdx.y * kArgmaxChunk, end = min(V, begin + kArgmaxChunk);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  if (((reinterpret_cast<uintptr_t>(row) | (uintptr_t)begin * 4) & 15) == 0 && end - begin == kArgmaxChunk) {
    // a whole chunk of an aligned row: 16 bytes a load, a thread's four loads asked for together
    float4 v[kArgmaxChunk / 4 / 256];
#pragma unroll
    for (int j = 0; j < kArgmaxChunk / 4 / 256; ++j)
      v[j] = __ldg(reinterpret_cast<const float4*>(row + begin) + j * 256 + threadIdx.x);
#pragma unroll
    for (int j = 0; j < kArgmaxChunk / 4 / 256; ++j) {
      const int i0 = begin + (j * 256 + (int)threadIdx.x) * 4;        // (indices rise: a later equal value never wins)
      const float e[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (e[k] > best) {
          best = e[k];
          bi = i0 + k;
        }
    }
  } else {
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
      const float v = row[i];
      if (v > best || (v == best && i < bi)) {
        best = v;
        bi = i;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sval[warp] = best;
    sidx[warp] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (sval[w] > best || (sval[w] == best && sidx[w] < bi)) {
        best = sval[w];
        bi = sidx[w];
      }
    cval[(size_t)blockIdx.x * n_chunks + blockIdx.y] = best;
    cidx[(size_t)blockIdx.x * n_chunks + blockIdx.y] = bi;
  }
}

__global__ void __launch_bounds__(32) argmax_final_kernel(const float* __restrict__ cval,
                                                         const int* __restrict__ cidx, int n_chunks,
                                                         int* __restrict__ out) {
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = threadIdx.x; c < n_chunks; c += 32) {
    const float v = cval[(size_t)blockIdx.x * n_chunks + c];
    const int i = cidx[(size_t)blockIdx.x * n_chunks + c];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if (threadIdx.x == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
}

// Block-wide deterministic sum of one float per thread; every thread gets the total.
__device__ __forceinline__ float block_total(float v, float* red) { return block_sum(v, red); }

__device__ __forceinline__ int block_count(int v, int* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  int total = 0;
  for (int w = 0; w < nwarp; ++w) total += red[w];
  return total;
}

// The fast way to a cut token set. A top-k or top-p cut keeps few tokens, all of them near the row's maximum, but
// finding the cut values by bisection takes some 30 passes each, and over the whole row (600 KB at a vocabulary of
// 152k) that is a millisecond. So: ONE pass counts the tokens within 1, 2, 3, 4, 6, 8, 12 and 16 of the maximum (in
// units of z) and sums the row's total weight; the widest of these bands that holds at most kCandidates tokens is
// copied to shared memory in index order (one more pass), and the bisections and the draw run there. That is exact
// as long as the cuts lie inside the band: a top-k beyond the band's tokens, or a nucleus that reaches below it,
// returns false, and the caller goes over the whole row as before. (Same rules, same ties: a token equal to a cut
// value is kept.) `*token` receives the choice (thread 0 writes it; the caller reads it behind a barrier).
constexpr int kCandidates = 4096;
constexpr int kBands = 8;

__device__ __forceinline__ float sample_band(int b) {
  return b == 0 ? 1.f : b == 1 ? 2.f : b == 2 ? 3.f : b == 3 ? 4.f : b == 4 ? 6.f : b == 5 ? 8.f : b == 6 ? 12.f : 16.f;
}

// Three block-wide sums at once, each taken exactly as block_sum takes one (so a sum does not depend on what it
// shares the pass with). `red` holds 3 x 32 floats.
__device__ __forceinline__ void block_sum3(float (&v)[3], float (*red)[32]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int j = 0; j < 3; ++j) v[j] = warp_sum(v[j]);
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int j = 0; j < 3; ++j) red[j][warp] = v[j];
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    float total = 0.f;
    for (int w = 0; w < nwarp; ++w) total += red[j][w];
    v[j] = total;
  }
}

// Three block-wide counts of at most 2^20 each, packed into one 64-bit sum.
__device__ __forceinline__ void block_count3(int (&c)[3], unsigned long long* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  unsigned long long v = (unsigned long long)c[0] | ((unsigned long long)c[1] << 21) | ((unsigned long long)c[2] << 42);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  unsigned long long total = 0;
  for (int w = 0; w < nwarp; ++w) total += red[w];
  c[0] = (int)(total & 0x1fffffull);
  c[1] = (int)((total >> 21) & 0x1fffffull);
  c[2] = (int)((total >> 42) & 0x1fffffull);
}

// The cuts and the draw among candidates in shared memory: cz / ci hold the n_cand tokens with z >= v0 in index
// order, all_mass the whole row's weight sum(exp(z - mx)). False when a cut lies below the candidates.
__device__ bool sample_among_candidates(const float* cz, const int* ci, int n_cand, float v0, float mx, float all_mass,
                                        int k, int V, float tp, float u, float* redf, int* redi, int* redi2,
                                        int* token) {
  __shared__ float red3[3][32];
  __shared__ unsigned long long red64[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
  // Top-k inside the band: the largest value v with count(z >= v) >= k.
  float cut = -INFINITY;
  if (k > 0 && k < V) {
    if (k > n_cand) return false;                            // the k-th token lies below the band
    unsigned int lo = float_order_bits(v0), hi = float_order_bits(mx);     // count(z >= v0) = n_cand >= k: the invariant
    // Three probes a pass cut the range in four (12 to 16 passes where halving takes 31): the counts are
    // monotone, so the largest probe that still has k tokens at or above it is the new lower end.
    while (lo < hi) {
      const unsigned long long span = hi - lo;
      unsigned int m[3];
      float v[3];
      int c[3] = {0, 0, 0};
#pragma unroll
      for (int q = 0; q < 3; ++q) {
        m[q] = lo + (unsigned int)((span * (q + 1) + 3ull) / 4ull);          // lo < m[0] <= m[1] <= m[2] <= hi
        v[q] = order_bits_float(m[q]);
      }
      for (int j = tid; j < n_cand; j += blockDim.x) {
        const float zv = cz[j];
#pragma unroll
        for (int q = 0; q < 3; ++q) c[q] += zv >= v[q] ? 1 : 0;
      }
      block_count3(c, red64);
      if (c[2] >= k) {
        lo = m[2];
      } else if (c[1] >= k) {
        lo = m[1];
        hi = m[2] - 1u;
      } else if (c[0] >= k) {
        lo = m[0];
        hi = m[1] - 1u;
      } else {
        hi = m[0] - 1u;
      }
    }
    cut = order_bits_float(lo);
  }
  // Top-p: the smallest x >= cut with mass(z > x) <= top_p * mass(kept so far); it must lie inside the band.
  if (tp < 1.0f) {
    float zk = all_mass;
    if (cut != -INFINITY) {
      zk = 0.f;
      for (int j = tid; j < n_cand; j += blockDim.x) zk += cz[j] >= cut ? expf(cz[j] - mx) : 0.f;
      zk = block_total(zk, redf);
    }
    const float budget = tp * zk;
    const float floor_x = fmaxf(cut, v0);
    float above = 0.f;                                       // mass(z > floor_x): must exceed the budget, or the
    for (int j = tid; j < n_cand; j += blockDim.x)           // nucleus reaches down to floor_x or below it
      above += (cz[j] > floor_x && cz[j] >= cut) ? expf(cz[j] - mx) : 0.f;
    above = block_total(above, redf);
    if (above <= budget) {
      if (cut == -INFINITY || cut < v0) return false;        // ... below the band: the whole row has to be read
      // (the cut itself is the answer: every token the top-k kept stays)
    } else {
      unsigned int lo = float_order_bits(floor_x), hi = float_order_bits(mx);   // predicate true at hi (mass 0)
      // Three probes a pass here too: the mass above a value falls as the value rises, so the smallest probe
      // whose mass fits the budget is the new upper end. (Each mass is summed as a pass of its own would.)
      while (lo < hi) {
        const unsigned long long span = hi - lo;
        unsigned int p[3];
        float x[3], m[3] = {0.f, 0.f, 0.f};
#pragma unroll
        for (int q = 0; q < 3; ++q) {
          p[q] = lo + (unsigned int)(span * (q + 1) / 4ull);                  // lo <= p[0] <= p[1] <= p[2] < hi
          x[q] = order_bits_float(p[q]);
        }
        for (int j = tid; j < n_cand; j += blockDim.x) {
          const float zv = cz[j];
          const float wgt = zv >= cut ? expf(zv - mx) : 0.f;
#pragma unroll
          for (int q = 0; q < 3; ++q) m[q] += zv > x[q] ? wgt : 0.f;
        }
        block_sum3(m, red3);
        if (m[0] <= budget) {
          hi = p[0];
        } else if (m[1] <= budget) {
          lo = p[0] + 1u;
          hi = p[1];
        } else if (m[2] <= budget) {
          lo = p[1] + 1u;
          hi = p[2];
        } else {
          lo = p[2] + 1u;
        }
      }
      cut = fmaxf(cut, order_bits_float(lo));
    }
  }
  if (cut == -INFINITY || cut < v0) return false;            // (no cut inside the band after all)

  // The draw: the first candidate, in index order, whose running sum of kept weights exceeds u * total. A thread
  // owns a contiguous run of candidates; the runs' sums meet in shared memory.
  const int per = (n_cand + (int)blockDim.x - 1) / (int)blockDim.x;
  const int j0 = min(n_cand, tid * per), j1 = min(n_cand, j0 + per);
  float mine = 0.f;
  for (int j = j0; j < j1; ++j) mine += cz[j] >= cut ? expf(cz[j] - mx) : 0.f;
  // exclusive prefix of `mine` over the threads, in thread order: warp scan, then the warps' totals
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  __syncthreads();
  if (lane == 31) redf[warp] = incl;
  __syncthreads();
  float before = 0.f, total = 0.f;
  for (int w = 0; w < nwarp; ++w) {
    if (w < warp) before += redf[w];
    total += redf[w];
  }
  before += incl - mine;
  const float target = u * total;
  int found = 0x7fffffff, last_kept = -1;
  float run = before;
  for (int j = j0; j < j1; ++j) {
    const float wgt = cz[j] >= cut ? expf(cz[j] - mx) : 0.f;
    if (wgt > 0.f) {
      last_kept = j;
      if (found == 0x7fffffff && target < run + wgt) found = j;
    }
    run += wgt;
  }
  // the lowest hit over the block; if u * total rounded up to the total, the last kept candidate
  __syncthreads();
  int best = found;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
  int lastk = last_kept;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lastk = max(lastk, __shfl_xor_sync(0xffffffffu, lastk, o));
  if (lane == 0) {
    redi[warp] = best;
    redi2[warp] = lastk;
  }
  __syncthreads();
  if (tid == 0) {
    int b = 0x7fffffff, l = -1;
    for (int w = 0; w < nwarp; ++w) {
      b = min(b, redi[w]);
      l = max(l, redi2[w]);
    }
    const int j = b != 0x7fffffff ? b : l;
    *token = j >= 0 ? ci[j] : -1;
  }
  __syncthreads();
  return true;
}

__device__ bool sample_from_candidates(const float* __restrict__ row, int V, float inv_t, float mx, int k, float tp,
                                       float u, float* redf, int* redi, int* token) {
  __shared__ float cz[kCandidates];
  __shared__ int ci[kCandidates];
  __shared__ int redi2[32];
  __shared__ int band_count[32][kBands];
  __shared__ float warp_mass[32];
  __shared__ int s_band;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
  const int span = (V + nwarp - 1) / nwarp;
  const int begin = warp * span, end = min(V, begin + span);

  // Pass 1: per warp span, how many tokens lie in each band, and the span's weight.
  int cnt[kBands];
#pragma unroll
  for (int b = 0; b < kBands; ++b) cnt[b] = 0;
  float mass = 0.f;
  float floor_of[kBands];                                    // a band's tokens: z >= mx - width, compared as floats
#pragma unroll
  for (int b = 0; b < kBands; ++b) floor_of[b] = mx - sample_band(b);
  for (int i = begin + lane; i < end; i += 32) {
    const float zv = row[i] * inv_t;
    mass += expf(zv - mx);
#pragma unroll
    for (int b = 0; b < kBands; ++b) cnt[b] += zv >= floor_of[b] ? 1 : 0;
  }
#pragma unroll
  for (int b = 0; b < kBands; ++b) {
    int c = cnt[b];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if (lane == 0) band_count[warp][b] = c;
  }
  mass = warp_sum(mass);
  if (lane == 0) warp_mass[warp] = mass;
  __syncthreads();
  if (tid == 0) {
    int chosen = -1;
    for (int b = 0; b < kBands; ++b) {
      int c = 0;
      for (int w = 0; w < nwarp; ++w) c += band_count[w][b];
      if (c <= kCandidates) chosen = b;
    }
    s_band = chosen;
  }
  __syncthreads();
  const int band = s_band;
  if (band < 0) return false;                                // more than kCandidates tokens within 1 of the maximum
  const float v0 = mx - sample_band(band);                   // candidates: z >= v0 (the comparison the counts used)
  float all_mass = 0.f;
  int offset = 0, n_cand = 0;
  for (int w = 0; w < nwarp; ++w) {
    all_mass += warp_mass[w];
    if (w < warp) offset += band_count[w][band];
    n_cand += band_count[w][band];
  }
  // Pass 2: the band's tokens to shared memory, in index order.
  for (int base = begin; base < end; base += 32) {
    const int i = base + lane;
    float zv = 0.f;
    bool in = false;
    if (i < end) {
      zv = row[i] * inv_t;
      in = zv >= v0;
    }
    const unsigned int ballot = __ballot_sync(0xffffffffu, in);
    if (in) {
      const int at = offset + __popc(ballot & ((1u << lane) - 1u));
      cz[at] = zv;
      ci[at] = i;
    }
    offset += __popc(ballot);
  }
  __syncthreads();
  return sample_among_candidates(cz, ci, n_cand, v0, mx, all_mass, k, V, tp, u, redf, redi, redi2, token);
}

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(
    const float* __restrict__ logits, int V, long long row_stride, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
    const int* __restrict__ rows, int* __restrict__ out, int scatter) {
  __shared__ float redf[32];
  __shared__ int redi[32];
  __shared__ float warp_tot[32];
  __shared__ int s_token;
  const int rowi = blockIdx.x;  // index into the parameter arrays and `out`
  const float* row = logits + (size_t)(rows ? rows[rowi] : rowi) * row_stride;
  const float inv_t = 1.0f / temperature[rowi];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;

  // Row maximum of z = logit / T.
  float mx = -INFINITY;
  for (int i = tid; i < V; i += blockDim.x) mx = fmaxf(mx, row[i] * inv_t);
  mx = warp_max(mx);
  __syncthreads();
  if (lane == 0) redf[warp] = mx;
  __syncthreads();
  mx = -INFINITY;
  for (int w = 0; w < nwarp; ++w) mx = fmaxf(mx, redf[w]);
  __syncthreads();

  const int k = top_k[rowi];
  const float tp = top_p[rowi];
  if (((k > 0 && k < V) || tp < 1.0f) &&
      sample_from_candidates(row, V, inv_t, mx, k, tp, uniform[rowi], redf, redi, &s_token)) {
    if (tid == 0) out[scatter && rows ? rows[rowi] : rowi] = s_token < 0 ? 0 : s_token;
    return;
  }
  __syncthreads();

  // The whole row, pass by pass (no cut asked for, or one that reaches below the candidates).
  // Cut value: keep z >= cut. Starts at "everything".
  float cut = -INFINITY;
  if (k > 0 && k < V) {
    // Largest value v with count(z >= v) >= k, by bisection on the ordered bit pattern.
    // Invariant: count(z >= value(lo)) >= k. It holds at -inf (every finite z counts); starting below
    // -inf would put NaN patterns, for which no comparison holds, inside the searched range.
    unsigned int lo = float_order_bits(-INFINITY), hi = float_order_bits(mx);
    while (lo < hi) {
      const unsigned int mid = lo + ((hi - lo + 1u) >> 1);
      const float v = order_bits_float(mid);
      int c = 0;
      for (int i = tid; i < V; i += blockDim.x) c += (row[i] * inv_t >= v) ? 1 : 0;
      c = block_count(c, redi);
      if (c >= k) lo = mid; else hi = mid - 1u;
    }
    cut = order_bits_float(lo);
  }
  if (tp < 1.0f) {
    float zk = 0.f;
    for (int i = tid; i < V; i += blockDim.x) {
      const float zv = row[i] * inv_t;
      zk += zv >= cut ? expf(zv - mx) : 0.f;
    }
    zk = block_total(zk, redf);
    const float budget = tp * zk;
    // Smallest x >= cut with mass(z > x) <= budget; kept = z >= x.
    unsigned int lo = float_order_bits(cut), hi = float_order_bits(mx);  // predicate true at hi (mass 0)
    while (lo < hi) {
      const unsigned int mid = lo + ((hi - lo) >> 1);
      const float x = order_bits_float(mid);
      float mass = 0.f;
      for (int i = tid; i < V; i += blockDim.x) {
        const float zv = row[i] * inv_t;
        mass += (zv > x && zv >= cut) ? expf(zv - mx) : 0.f;
      }
      mass = block_total(mass, redf);
      if (mass <= budget) hi = mid; else lo = mid + 1u;
    }
    cut = fmaxf(cut, order_bits_float(lo));
  }

  // Inverse CDF in index order. Warp w owns the contiguous span [w * span, (w + 1) * span).
  const int span = (V + nwarp - 1) / nwarp;
  const int begin = warp * span, end = min(V, begin + span);
  float part = 0.f;
  for (int i = begin + lane; i < end; i += 32) {
    const float zv = row[i] * inv_t;
    part += zv >= cut ? expf(zv - mx) : 0.f;
  }
  part = warp_sum(part);
  if (lane == 0) warp_tot[warp] = part;
  if (tid == 0) s_token = -1;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarp; ++w) total += warp_tot[w];
  const float target = uniform[rowi] * total;
  float before = 0.f;
  int owner = -1;
  for (int w = 0; w < nwarp; ++w) {
    if (target < before + warp_tot[w]) {
      owner = w;
      break;
    }
    before += warp_tot[w];
  }
  if (owner < 0) {  // u * total rounded up to the total: the last warp with any weight owns it
    before = 0.f;
    for (int w = 0; w < nwarp; ++w) {
      if (warp_tot[w] > 0.f) owner = w;
    }
    for (int w = 0; w < owner; ++w) before += warp_tot[w];
  }
  if (warp == owner) {
    float run = before;
    int found = -1, last_kept = -1;
    for (int base = begin; base < end && found < 0; base += 32) {
      const int i = base + lane;
      float wgt = 0.f;
      if (i < end) {
        const float zv = row[i] * inv_t;
        wgt = zv >= cut ? expf(zv - mx) : 0.f;
      }
      float incl = wgt;  // inclusive scan over the 32 lanes
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
      }
      const bool hit = wgt > 0.f && target < run + incl;
      const unsigned int ballot = __ballot_sync(0xffffffffu, hit);
      const unsigned int kept = __ballot_sync(0xffffffffu, wgt > 0.f);
      if (kept) last_kept = base + (31 - __clz(kept));
      if (ballot) found = base + (__ffs(ballot) - 1);
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) s_token = found >= 0 ? found : last_kept;
  }
  __syncthreads();
  if (tid == 0) out[scatter && rows ? rows[rowi] : rowi] = s_token < 0 ? 0 : s_token;
}


// ---- A row over a cluster of blocks -------------------------------------------------------------------------
// One block per row reads 600 KB alone at a vocabulary of 152k, once per pass. Here a cluster of eight blocks
// takes a row: each block copies an eighth of it to its shared memory once (z = logit / T), every later pass runs
// there, and what the blocks have to tell each other (the maximum, counts, sums) goes through distributed shared
// memory: a block writes its few words into every block's table and arrives on every block's mbarrier; a block
// goes on when all eight have arrived on its own. Sums are taken in thread order inside a block and in rank
// order across blocks, so the result does not depend on timing. The rules are the ones above (same cuts, same
// ties, same inverse-CDF walk in index order); candidates go to the first block's shared memory.
// Every wait is bounded; a block that gives up raises the error word, and all blocks meet at the cluster's
// hardware barrier before they leave, so none leaves while another may still write to it.
constexpr int kClusterBlocks = 8;
constexpr int kClusterThreads = 512;
constexpr int kClusterWarps = kClusterThreads / 32;
constexpr int kClusterVals = 12;             // 32-bit words a block hands to the others in one round
constexpr uint32_t kClusterSpin = 1u << 22;
constexpr int kClusterMinVocab = 8192;            // narrower rows stay with one block
constexpr int kClusterMaxSliceBytes = 160 * 1024;  // a block's slice of a row (a vocabulary of up to 327k)

__device__ __forceinline__ uint32_t sm_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_addr(uint32_t addr, uint32_t rank) {   // the same variable in another block
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_store(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

struct ClusterComm {
  uint32_t bar;        // this block's two mbarriers (shared-memory address): rounds alternate between them
  uint32_t table;      // this block's table [2][kClusterBlocks][kClusterVals] (shared-memory address)
  const uint32_t* got; // the same table through a generic pointer
  uint32_t* mine;      // [kClusterVals]: what this block hands out in the next round
  uint32_t rank;
  unsigned round;
  int* error;
};

// One round: words mine[0 .. n) of every block land in row `rank` of every block's table; returns that table
// (row r = block r's words) once all blocks have arrived, or null when the wait ran out (same answer in every
// thread of the block). Two tables and two mbarriers alternate: a block can be one round ahead of another,
// never two, so an arrival for the round after next cannot be counted with this round's.
__device__ __forceinline__ const uint32_t* cluster_round(ClusterComm& c, int n) {
  const int tid = threadIdx.x;
  const unsigned b = c.round & 1u;
  __syncthreads();                                           // mine[] is complete
  if (tid < kClusterBlocks * n) {
    const int dst = tid / n, idx = tid - dst * n;
    cluster_store(cluster_addr(c.table + ((b * kClusterBlocks + c.rank) * kClusterVals + idx) * 4u, dst), c.mine[idx]);
  }
  asm volatile("fence.acq_rel.cluster;" ::: "memory");       // (the candidates' stores of a round without words too)
  __syncthreads();                                           // this block's stores come before its arrivals
  const uint32_t bar = c.bar + b * 8u, parity = (c.round >> 1) & 1u;
  if (tid < kClusterBlocks)
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr(bar, tid)) : "memory");
  uint32_t spins = 0, done = 0;
  while (!done) {
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (!done && ++spins > kClusterSpin) break;
  }
  const int bad = __syncthreads_or(done ? 0 : 1);
  c.round += 1;
  if (bad) {
    if (tid == 0) atomicCAS(c.error, 0, 41);
    return nullptr;
  }
  return c.got + (size_t)b * kClusterBlocks * kClusterVals;
}

// The token at which the running sum of kept weights (z >= cut), in index order over this block's slice, passes
// `target`; `before` is the sum over the blocks in front. warp_tot: the kept weight of each warp's span (already
// there). When the target lies beyond everything (u * total rounded up to the total) the last kept token.
__device__ __forceinline__ void cluster_draw_in_block(const float* zs, int n, int index0, float cut, float mx,
                                                      float target, float before, const float* warp_tot, int* s_token) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int span = (n + kClusterWarps - 1) / kClusterWarps;
  const int begin = min(n, warp * span), end = min(n, begin + span);
  int owner = -1;
  float run0 = before;
  for (int w = 0; w < kClusterWarps; ++w) {
    if (target < run0 + warp_tot[w]) {
      owner = w;
      break;
    }
    run0 += warp_tot[w];
  }
  if (owner < 0) {
    run0 = before;
    for (int w = 0; w < kClusterWarps; ++w)
      if (warp_tot[w] > 0.f) owner = w;
    for (int w = 0; w < owner; ++w) run0 += warp_tot[w];
  }
  if (tid == 0) *s_token = -1;
  __syncthreads();
  if (warp == owner) {
    float run = run0;
    int found = -1, last_kept = -1;
    for (int base = begin; base < end && found < 0; base += 32) {
      const int j = base + lane;
      float wgt = 0.f;
      if (j < end) wgt = zs[j] >= cut ? expf(zs[j] - mx) : 0.f;
      float incl = wgt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      const unsigned int hit = __ballot_sync(0xffffffffu, wgt > 0.f && target < run + incl);
      const unsigned int kept = __ballot_sync(0xffffffffu, wgt > 0.f);
      if (kept) last_kept = base + (31 - __clz(kept));
      if (hit) found = base + (__ffs(hit) - 1);
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) *s_token = index0 + (found >= 0 ? found : last_kept);
  }
  __syncthreads();
}

__device__ __forceinline__ void sample_cluster_body(ClusterComm& c, const float* zs, int n, int index0, int V, float mx_local,
                                                    int k, float tp, float u, float* cz, int* ci, float* redf, int* redi,
                                                    int* redi2, int (*band_count)[kBands], float* warp_tot,
                                                    int* s_token, int* out_slot) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int span = (n + kClusterWarps - 1) / kClusterWarps;
  const int begin = min(n, warp * span), end = min(n, begin + span);      // this warp's contiguous span of the slice
  // The row's maximum.
  if (tid == 0) c.mine[0] = __float_as_uint(mx_local);
  const uint32_t* got = cluster_round(c, 1);
  if (!got) return;
  float mx = -INFINITY;
  for (int r = 0; r < kClusterBlocks; ++r) mx = fmaxf(mx, __uint_as_float(got[r * kClusterVals]));

  float cut = -INFINITY;
  const bool has_k = k > 0 && k < V;
  if (has_k || tp < 1.0f) {
    // The candidates: counts per band and the weight of each warp's span; the blocks' sums go round.
    int cnt[kBands];
    float floor_of[kBands];
#pragma unroll
    for (int b = 0; b < kBands; ++b) {
      cnt[b] = 0;
      floor_of[b] = mx - sample_band(b);
    }
    float mass = 0.f;
    for (int j = begin + lane; j < end; j += 32) {
      const float zv = zs[j];
      mass += expf(zv - mx);
#pragma unroll
      for (int b = 0; b < kBands; ++b) cnt[b] += zv >= floor_of[b] ? 1 : 0;
    }
#pragma unroll
    for (int b = 0; b < kBands; ++b) {
      int v = cnt[b];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) band_count[warp][b] = v;
    }
    mass = warp_sum(mass);
    if (lane == 0) warp_tot[warp] = mass;
    __syncthreads();
    if (tid < kBands) {
      int v = 0;
      for (int w = 0; w < kClusterWarps; ++w) v += band_count[w][tid];
      c.mine[tid] = (uint32_t)v;
    }
    if (tid == kBands) {
      float m = 0.f;
      for (int w = 0; w < kClusterWarps; ++w) m += warp_tot[w];
      c.mine[kBands] = __float_as_uint(m);
    }
    got = cluster_round(c, kBands + 1);
    if (!got) return;
    int band = -1;
    for (int b = 0; b < kBands; ++b) {
      int v = 0;
      for (int r = 0; r < kClusterBlocks; ++r) v += (int)got[r * kClusterVals + b];
      if (v <= kCandidates) band = b;
    }
    if (band >= 0) {
      float all_mass = 0.f;
      int offset = 0, n_cand = 0;
      for (int r = 0; r < kClusterBlocks; ++r) {
        all_mass += __uint_as_float(got[r * kClusterVals + kBands]);
        const int v = (int)got[r * kClusterVals + band];
        if (r < (int)c.rank) offset += v;
        n_cand += v;
      }
      for (int w = 0; w < warp; ++w) offset += band_count[w][band];
      const float v0 = mx - sample_band(band);
      // The band's tokens into the first block's shared memory, in index order.
      const uint32_t cz0 = cluster_addr(sm_addr(cz), 0), ci0 = cluster_addr(sm_addr(ci), 0);
      for (int base = begin; base < end; base += 32) {
        const int j = base + lane;
        float zv = 0.f;
        bool in = false;
        if (j < end) {
          zv = zs[j];
          in = zv >= v0;
        }
        const unsigned int ballot = __ballot_sync(0xffffffffu, in);
        if (in) {
          const int at = offset + __popc(ballot & ((1u << lane) - 1u));
          cluster_store(cz0 + at * 4u, __float_as_uint(zv));
          cluster_store(ci0 + at * 4u, (uint32_t)(index0 + j));
        }
        offset += __popc(ballot);
      }
      if (!cluster_round(c, 0)) return;                      // every block's candidates are in place
      if (c.rank == 0) {
        const bool done = sample_among_candidates(cz, ci, n_cand, v0, mx, all_mass, k, V, tp, u, redf, redi, redi2, s_token);
        if (tid == 0) {
          c.mine[0] = done ? 1u : 0u;
          if (done) *out_slot = *s_token < 0 ? 0 : *s_token;
        }
      } else if (tid == 0) {
        c.mine[0] = 0u;
      }
      got = cluster_round(c, 1);
      if (!got) return;
      if (got[0]) return;                                    // the first block has drawn
    }
    // A cut below the candidates: the bisections over the whole row, a round of the cluster per step.
    if (has_k) {
      unsigned int lo = float_order_bits(-INFINITY), hi = float_order_bits(mx);
      while (lo < hi) {
        const unsigned int mid = lo + ((hi - lo + 1u) >> 1);
        const float v = order_bits_float(mid);
        int cn = 0;
        for (int j = tid; j < n; j += kClusterThreads) cn += zs[j] >= v ? 1 : 0;
        cn = block_count(cn, redi);
        if (tid == 0) c.mine[0] = (uint32_t)cn;
        got = cluster_round(c, 1);
        if (!got) return;
        int all = 0;
        for (int r = 0; r < kClusterBlocks; ++r) all += (int)got[r * kClusterVals];
        if (all >= k) lo = mid; else hi = mid - 1u;
      }
      cut = order_bits_float(lo);
    }
    if (tp < 1.0f) {
      auto mass_above = [&](float x, bool strictly) -> float {     // kept weight above x, over the whole row
        float m = 0.f;
        for (int j = tid; j < n; j += kClusterThreads) {
          const float zv = zs[j];
          m += ((strictly ? zv > x : true) && zv >= cut) ? expf(zv - mx) : 0.f;
        }
        m = block_total(m, redf);
        if (tid == 0) c.mine[0] = __float_as_uint(m);
        const uint32_t* g = cluster_round(c, 1);
        if (!g) return -1.f;
        float all = 0.f;
        for (int r = 0; r < kClusterBlocks; ++r) all += __uint_as_float(g[r * kClusterVals]);
        return all;
      };
      const float zk = mass_above(0.f, false);
      if (zk < 0.f) return;
      const float budget = tp * zk;
      unsigned int lo = float_order_bits(cut), hi = float_order_bits(mx);   // predicate true at hi (mass 0)
      while (lo < hi) {
        const unsigned int mid = lo + ((hi - lo) >> 1);
        const float m = mass_above(order_bits_float(mid), true);
        if (m < 0.f) return;
        if (m <= budget) hi = mid; else lo = mid + 1u;
      }
      cut = fmaxf(cut, order_bits_float(lo));
    }
  }

  // The draw over the whole row: the kept weight of every warp's span, of every block, then the walk in the
  // block the target falls into.
  float part = 0.f;
  for (int j = begin + lane; j < end; j += 32) part += zs[j] >= cut ? expf(zs[j] - mx) : 0.f;
  part = warp_sum(part);
  __syncthreads();
  if (lane == 0) warp_tot[warp] = part;
  __syncthreads();
  if (tid == 0) {
    float m = 0.f;
    for (int w = 0; w < kClusterWarps; ++w) m += warp_tot[w];
    c.mine[0] = __float_as_uint(m);
  }
  got = cluster_round(c, 1);
  if (!got) return;
  float total = 0.f;
  for (int r = 0; r < kClusterBlocks; ++r) total += __uint_as_float(got[r * kClusterVals]);
  const float target = u * total;
  int owner = -1;
  float before = 0.f;
  for (int r = 0; r < kClusterBlocks; ++r) {
    const float m = __uint_as_float(got[r * kClusterVals]);
    if (target < before + m) {
      owner = r;
      break;
    }
    before += m;
  }
  if (owner < 0) {                                           // u * total rounded up to the total
    before = 0.f;
    for (int r = 0; r < kClusterBlocks; ++r)
      if (__uint_as_float(got[r * kClusterVals]) > 0.f) owner = r;
    for (int r = 0; r < owner; ++r) before += __uint_as_float(got[r * kClusterVals]);
  }
  if ((int)c.rank == owner) {
    cluster_draw_in_block(zs, n, index0, cut, mx, target, before, warp_tot, s_token);
    if (tid == 0) *out_slot = *s_token < 0 ? 0 : *s_token;
  }
}

__global__ void __cluster_dims__(kClusterBlocks, 1, 1) __launch_bounds__(kClusterThreads) sample_cluster_kernel(
    const float* __restrict__ logits, int V, long long row_stride, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
    const int* __restrict__ rows, int* __restrict__ out, int scatter, int per, int vec, int* error) {
  extern __shared__ __align__(16) float zs[];                // this block's slice of z = logit / T
  __shared__ float cz[kCandidates];
  __shared__ int ci[kCandidates];
  __shared__ uint32_t table[2][kClusterBlocks][kClusterVals];
  __shared__ uint32_t mine[kClusterVals];
  __shared__ __align__(8) unsigned long long bar[2];
  __shared__ float redf[32];
  __shared__ int redi[32], redi2[32];
  __shared__ int band_count[kClusterWarps][kBands];
  __shared__ float warp_tot[kClusterWarps];
  __shared__ int s_token;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t rank = cluster_rank();
  const int rowi = blockIdx.x / kClusterBlocks;
  const float* row = logits + (size_t)(rows ? rows[rowi] : rowi) * row_stride;
  const float inv_t = 1.0f / temperature[rowi];
  const int index0 = min(V, (int)rank * per), n = min(V, index0 + per) - index0;
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sm_addr(&bar[0])), "r"(kClusterBlocks));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sm_addr(&bar[1])), "r"(kClusterBlocks));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // The slice, once, and its maximum.
  float mx = -INFINITY;
  if (vec) {
    const float4* src = reinterpret_cast<const float4*>(row + index0);
    for (int j = tid; j < n / 4; j += kClusterThreads) {
      float4 v = __ldg(src + j);
      v.x *= inv_t; v.y *= inv_t; v.z *= inv_t; v.w *= inv_t;
      *reinterpret_cast<float4*>(zs + 4 * j) = v;
      mx = fmaxf(fmaxf(mx, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
    }
    for (int j = n / 4 * 4 + tid; j < n; j += kClusterThreads) {
      const float v = row[index0 + j] * inv_t;
      zs[j] = v;
      mx = fmaxf(mx, v);
    }
  } else {
    for (int j = tid; j < n; j += kClusterThreads) {
      const float v = row[index0 + j] * inv_t;
      zs[j] = v;
      mx = fmaxf(mx, v);
    }
  }
  mx = warp_max(mx);
  if (lane == 0) redf[warp] = mx;
  __syncthreads();
  mx = -INFINITY;
  for (int w = 0; w < kClusterWarps; ++w) mx = fmaxf(mx, redf[w]);
  __syncthreads();
  cluster_sync_all();                                        // every block's mbarrier is ready before anyone arrives on it
  ClusterComm c{sm_addr(&bar[0]), sm_addr(&table[0][0][0]), &table[0][0][0], mine, rank, 0u, error};
  sample_cluster_body(c, zs, n, index0, V, mx, top_k[rowi], top_p[rowi], uniform[rowi], cz, ci, redf, redi, redi2,
                      band_count, warp_tot, &s_token, out + (scatter && rows ? rows[rowi] : rowi));
  cluster_sync_all();                                        // nobody leaves while another may still write to it
}

}  // namespace tmk

// How many chunks tm_argmax cuts a row of V logits into (scratch: n_rows * chunks floats and ints).
extern "C" int tm_argmax_chunks(int V) { return (V + tmk::kArgmaxChunk - 1) / tmk::kArgmaxChunk; }

// scratch_val / scratch_idx: [n_rows, tm_argmax_chunks(V)] (may be null when V fits one chunk).
extern "C" int tm_argmax(const float* logits, int n_rows, int V, long long row_stride, int* out,
                         float* scratch_val, int* scratch_idx, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (V <= 0) return TM_ERR_UNSUPPORTED_SHAPE;
  const int chunks = tm_argmax_chunks(V);
  if (chunks <= 1) {
    tmk::argmax_kernel<<<n_rows, tmk::kSampleThreads, 0, stream>>>(logits, V, row_stride, out);
    return tmk::launch_status();
  }
  if (!scratch_val || !scratch_idx) return TM_ERR_SCRATCH_TOO_SMALL;
  tmk::argmax_chunk_kernel<<<dim3(n_rows, chunks), 256, 0, stream>>>(logits, V, row_stride, scratch_val,
                                                                    scratch_idx, chunks);
  tmk::argmax_final_kernel<<<n_rows, 32, 0, stream>>>(scratch_val, scratch_idx, chunks, out);
  return tmk::launch_status();
}

// temperature [n] (> 0), top_k [n] (<= 0 or >= V: off), top_p [n] (>= 1: off), uniform [n] in [0, 1).
// rows [n] (or null): which row of `logits` draw i reads; out [n], or with `scatter` an array indexed like the
// logits rows: draw i then lands in out[rows[i]] (the other entries stay as they are).
extern "C" int tm_sample(const float* logits, int n_rows, int V, long long row_stride, const float* temperature,
                         const int* top_k, const float* top_p, const float* uniform, const int* rows, int* out,
                         int scatter, int* error, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (V <= 0) return TM_ERR_UNSUPPORTED_SHAPE;
  // A wide row goes over a cluster of blocks, an eighth of it in each block's shared memory (`error`: the
  // device word a block raises when its wait for the others runs out; without one the single-block kernel runs).
  const int per = ((V + tmk::kClusterBlocks - 1) / tmk::kClusterBlocks + 3) / 4 * 4;
  if (error && V >= tmk::kClusterMinVocab && per * (int)sizeof(float) <= tmk::kClusterMaxSliceBytes) {
    static bool prepared = false;
    if (!prepared) {
      cudaError_t e = cudaFuncSetAttribute(tmk::sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           tmk::kClusterMaxSliceBytes);
      if (e != cudaSuccess) return (int)e;
      prepared = true;
    }
    const int vec = (reinterpret_cast<uintptr_t>(logits) % 16 == 0 && row_stride % 4 == 0) ? 1 : 0;
    tmk::sample_cluster_kernel<<<n_rows * tmk::kClusterBlocks, tmk::kClusterThreads, per * sizeof(float), stream>>>(
        logits, V, row_stride, temperature, top_k, top_p, uniform, rows, out, scatter, per, vec, error);
    if (cudaGetLastError() == cudaSuccess) return 0;
    // (A device that cannot place the cluster refuses the launch; the rows then go to one block each. An error
    // that is not about the launch shows again below.)
  }
  tmk::sample_kernel<<<n_rows, tmk::kSampleThreads, 0, stream>>>(logits, V, row_stride, temperature, top_k, top_p,
                                                              uniform, rows, out, scatter);
  return tmk::launch_status();
}
