// Token selection from 32-bit logits, one block per row.
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
// vocabulary of 152k), and over the whole row otherwise (1 to 1.7 ms).
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

__device__ bool sample_from_candidates(const float* __restrict__ row, int V, float inv_t, float mx, int k, float tp,
                                       float u, float* redf, int* redi, int* token) {
  __shared__ float cz[kCandidates];
  __shared__ int ci[kCandidates];
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

  // Top-k inside the band: the largest value v with count(z >= v) >= k.
  float cut = -INFINITY;
  if (k > 0 && k < V) {
    if (k > n_cand) return false;                            // the k-th token lies below the band
    unsigned int lo = float_order_bits(v0), hi = float_order_bits(mx);     // count(z >= v0) = n_cand >= k: the invariant
    while (lo < hi) {
      const unsigned int mid = lo + ((hi - lo + 1u) >> 1);
      const float v = order_bits_float(mid);
      int c = 0;
      for (int j = tid; j < n_cand; j += blockDim.x) c += cz[j] >= v ? 1 : 0;
      c = block_count(c, redi);
      if (c >= k) lo = mid; else hi = mid - 1u;
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
      while (lo < hi) {
        const unsigned int mid = lo + ((hi - lo) >> 1);
        const float x = order_bits_float(mid);
        float m = 0.f;
        for (int j = tid; j < n_cand; j += blockDim.x) m += (cz[j] > x && cz[j] >= cut) ? expf(cz[j] - mx) : 0.f;
        m = block_total(m, redf);
        if (m <= budget) hi = mid; else lo = mid + 1u;
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
    band_count[warp][0] = lastk;
  }
  __syncthreads();
  if (tid == 0) {
    int b = 0x7fffffff, l = -1;
    for (int w = 0; w < nwarp; ++w) {
      b = min(b, redi[w]);
      l = max(l, band_count[w][0]);
    }
    const int j = b != 0x7fffffff ? b : l;
    *token = j >= 0 ? ci[j] : -1;
  }
  __syncthreads();
  return true;
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
                         int scatter, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (V <= 0) return TM_ERR_UNSUPPORTED_SHAPE;
  tmk::sample_kernel<<<n_rows, tmk::kSampleThreads, 0, stream>>>(logits, V, row_stride, temperature, top_k, top_p,
                                                              uniform, rows, out, scatter);
  return tmk::launch_status();
}
