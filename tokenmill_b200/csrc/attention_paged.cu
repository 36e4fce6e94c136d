// Causal grouped-query attention over the paged cache, for any mix of prompt portions and single
// decoded tokens in one launch. 32-bit arithmetic on CUDA cores; it is the 32-bit path's attention and
// the fallback shape-generic kernel of the bfloat16 path (any head_dim that is a multiple of 16 up to
// 256, any head and group counts, any page size).
//
// Semantics (src/infer/model/layers.py:72-124, src/infer/kv/context.py:63-80): the step's keys and
// values are already in the cache; a query at absolute position p of its request reads keys j <= p
// of that request (and j > p - window if a window is set); S = q.k * scale; P = softmax(S) in
// 32-bit; O = P.V. Grouped-query attention: query head h reads kv head h / G.
//
// Work split: a tile is 32 consecutive (token, head-in-group) rows of one request and one kv head;
// 8 warps x 4 rows. Keys are walked in tiles of 32 anchored at absolute positions 0, 32, 64, ..., so
// the order of every sum depends only on the query's own position, never on how the request was cut
// into steps or on what else is in the batch. With split_keys > 0 the key range is also cut at
// absolute multiples of split_keys across blockIdx.z, partial (max, sum, acc) go to scratch, and
// tm_attention_combine merges them in index order.
#include "common.cuh"

namespace tmk {

constexpr int kRowsPerWarp = 4;
constexpr int kWarps = 8;
constexpr int kTileRows = kRowsPerWarp * kWarps;  // 32
constexpr int kKeyTile = 32;

template <typename T, int ND>  // ND = ceil(D / 32)
__global__ void __launch_bounds__(kWarps * 32) paged_attention_kernel(
    const T* __restrict__ q, const T* __restrict__ kcache, const T* __restrict__ vcache,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ cu_q,
    const int* __restrict__ kv_before, const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
    T* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml, int nh, int nkv, int D,
    int page_size, float scale, int window, int split_keys, int max_splits) {
  extern __shared__ __align__(16) float smem[];
  const int KS = D + 4;                    // padded row stride (floats) of the K tile: conflict-free float4 reads
  float* qs = smem;                        // [32][D]
  float* ks = qs + kTileRows * D;          // [32][D + 4]
  float* vs = ks + kKeyTile * KS;          // [32][D]

  const int G = nh / nkv;
  const int s = tile_seq[blockIdx.x];
  const int row0 = tile_row0[blockIdx.x];
  const int kvh = blockIdx.y;
  const int z = blockIdx.z;
  const int q_start = cu_q[s];
  const int q_len = cu_q[s + 1] - q_start;
  const int before = kv_before[s];
  const int n_rows = q_len * G;
  if (row0 >= n_rows) return;
  const int row_end = min(row0 + kTileRows, n_rows);
  const int p_min = before + row0 / G;
  const int p_max = before + (row_end - 1) / G;
  int j_lo = window > 0 ? max(0, p_min - window + 1) : 0;
  int j_hi = p_max;
  if (split_keys > 0) {
    j_lo = max(j_lo, z * split_keys);
    j_hi = min(j_hi, (z + 1) * split_keys - 1);
  }
  if (j_lo > j_hi) return;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* table = block_table + (size_t)s * bt_stride;

  // Stage the tile's queries in 32-bit.
  for (int idx = tid; idx < kTileRows * D; idx += blockDim.x) {
    const int r = idx / D, d = idx - r * D;
    const int row = row0 + r;
    float v = 0.f;
    if (row < n_rows) {
      const int tok = q_start + row / G, head = kvh * G + row % G;
      v = to_float(q[((size_t)tok * nh + head) * D + d]);
    }
    qs[idx] = v;
  }

  float m[kRowsPerWarp], l[kRowsPerWarp], acc[kRowsPerWarp][ND];
  int p_row[kRowsPerWarp], lo_row[kRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int dd = 0; dd < ND; ++dd) acc[i][dd] = 0.f;
    const int row = row0 + warp * kRowsPerWarp + i;
    if (row < n_rows) {
      p_row[i] = before + row / G;
      lo_row[i] = window > 0 ? max(0, p_row[i] - window + 1) : 0;
    } else {
      p_row[i] = -1;  // no key passes j <= -1: the row stays empty
      lo_row[i] = 0;
    }
  }

  const int D4 = D >> 2;
  for (int kt = (j_lo / kKeyTile) * kKeyTile; kt <= j_hi; kt += kKeyTile) {
    __syncthreads();  // previous tile fully consumed (and qs visible on the first trip)
    for (int idx = tid; idx < kKeyTile * D4; idx += blockDim.x) {
      const int jj = idx / D4, d4 = idx - jj * D4;
      const int j = kt + jj;
      float k4[4] = {0.f, 0.f, 0.f, 0.f}, v4[4] = {0.f, 0.f, 0.f, 0.f};
      if (j >= j_lo && j <= j_hi) {
        const int page = table[j / page_size];
        const size_t base = (((size_t)page * page_size + (j % page_size)) * nkv + kvh) * D + d4 * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          k4[e] = to_float(kcache[base + e]);
          v4[e] = to_float(vcache[base + e]);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        ks[jj * KS + d4 * 4 + e] = k4[e];
        vs[jj * D + d4 * 4 + e] = v4[e];
      }
    }
    __syncthreads();

    // Scores: lane j holds key kt + j for each of the warp's rows.
    float sc[kRowsPerWarp];
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) sc[i] = 0.f;
    const float4* krow = reinterpret_cast<const float4*>(ks + lane * KS);
    for (int d4 = 0; d4 < D4; ++d4) {
      const float4 kk = krow[d4];
#pragma unroll
      for (int i = 0; i < kRowsPerWarp; ++i) {
        const float4 qq = reinterpret_cast<const float4*>(qs + (warp * kRowsPerWarp + i) * D)[d4];
        sc[i] = fmaf(qq.x, kk.x, sc[i]);
        sc[i] = fmaf(qq.y, kk.y, sc[i]);
        sc[i] = fmaf(qq.z, kk.z, sc[i]);
        sc[i] = fmaf(qq.w, kk.w, sc[i]);
      }
    }
    const int j = kt + lane;
    float p[kRowsPerWarp];
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) {
      const bool ok = j >= j_lo && j <= j_hi && j <= p_row[i] && j >= lo_row[i];
      const float sv = ok ? sc[i] * scale : -INFINITY;
      const float tmax = warp_max(sv);
      const float m_new = fmaxf(m[i], tmax);
      float corr = 1.f, pv = 0.f;
      if (m_new != -INFINITY) {
        corr = expf(m[i] - m_new);  // m = -inf gives 0
        pv = ok ? expf(sv - m_new) : 0.f;
      }
      const float tsum = warp_sum(pv);
      l[i] = l[i] * corr + tsum;
      m[i] = m_new;
      p[i] = pv;
#pragma unroll
      for (int dd = 0; dd < ND; ++dd) acc[i][dd] *= corr;
    }
    // O += P.V : lane owns dims lane, lane + 32, ...
    for (int jj = 0; jj < kKeyTile; ++jj) {
      float vv[ND];
#pragma unroll
      for (int dd = 0; dd < ND; ++dd) {
        const int d = lane + 32 * dd;
        vv[dd] = d < D ? vs[jj * D + d] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < kRowsPerWarp; ++i) {
        const float pj = __shfl_sync(0xffffffffu, p[i], jj);
#pragma unroll
        for (int dd = 0; dd < ND; ++dd) acc[i][dd] = fmaf(pj, vv[dd], acc[i][dd]);
      }
    }
  }

#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    const int row = row0 + warp * kRowsPerWarp + i;
    if (row >= n_rows) continue;
    const int tok = q_start + row / G, head = kvh * G + row % G;
    const size_t orow = (size_t)tok * nh + head;
    if (split_keys > 0) {
      float* pa = part_acc + (orow * max_splits + z) * D;
#pragma unroll
      for (int dd = 0; dd < ND; ++dd) {
        const int d = lane + 32 * dd;
        if (d < D) pa[d] = acc[i][dd];
      }
      if (lane == 0) {
        part_ml[(orow * max_splits + z) * 2 + 0] = m[i];
        part_ml[(orow * max_splits + z) * 2 + 1] = l[i];
      }
    } else {
      const float inv = 1.0f / l[i];
#pragma unroll
      for (int dd = 0; dd < ND; ++dd) {
        const int d = lane + 32 * dd;
        if (d < D) out[orow * D + d] = from_float<T>(acc[i][dd] * inv);
      }
    }
  }
}

// One warp per (token, head) row: merge the row's partials, split index ascending.
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                         const int* __restrict__ cu_q, const int* __restrict__ kv_before,
                                         const int* __restrict__ seq_of_token, T* __restrict__ out, int n_tokens,
                                         int nh, int D, int window, int split_keys, int max_splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_tokens * nh) return;
  const int tok = row / nh;
  const int s = seq_of_token[tok];
  const int p = kv_before[s] + (tok - cu_q[s]);
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int z0 = lo / split_keys, z1 = p / split_keys;
  float mx = -INFINITY;
  for (int z = z0; z <= z1; ++z) mx = fmaxf(mx, part_ml[((size_t)row * max_splits + z) * 2]);
  float lsum = 0.f;
  for (int z = z0; z <= z1; ++z) {
    const float* ml = part_ml + ((size_t)row * max_splits + z) * 2;
    lsum += ml[1] * expf(ml[0] - mx);
  }
  const float inv = 1.0f / lsum;
  for (int d = lane; d < D; d += 32) {
    float a = 0.f;
    for (int z = z0; z <= z1; ++z) {
      const float w = expf(part_ml[((size_t)row * max_splits + z) * 2] - mx);
      a = fmaf(part_acc[((size_t)row * max_splits + z) * D + d], w, a);
    }
    out[(size_t)row * D + d] = from_float<T>(a * inv);
  }
}

template <typename T>
int launch_paged_attention(const void* q, const void* kcache, const void* vcache, const int* block_table,
                           int bt_stride, const int* cu_q, const int* kv_before, const int* tile_seq,
                           const int* tile_row0, int n_tiles, void* out, float* part_acc, float* part_ml, int nh,
                           int nkv, int D, int page_size, float scale, int window, int split_keys, int max_splits,
                           cudaStream_t stream) {
  const size_t smem = ((size_t)kTileRows * D + (size_t)kKeyTile * (D + 4) + (size_t)kKeyTile * D) * sizeof(float);
  const int nd = (D + 31) / 32;
  const dim3 grid(n_tiles, nkv, split_keys > 0 ? max_splits : 1);
#define TM_ATTN_CASE(NDV)                                                                                     \
  case NDV: {                                                                                                 \
    auto kern = paged_attention_kernel<T, NDV>;                                                               \
    if (smem > 48 * 1024) {                                                                                   \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
      if (e != cudaSuccess) return (int)e;                                                                    \
    }                                                                                                         \
    kern<<<grid, kWarps * 32, smem, stream>>>((const T*)q, (const T*)kcache, (const T*)vcache, block_table,   \
                                              bt_stride, cu_q, kv_before, tile_seq, tile_row0, (T*)out,       \
                                              part_acc, part_ml, nh, nkv, D, page_size, scale, window,        \
                                              split_keys, max_splits);                                        \
    break;                                                                                                    \
  }
  switch (nd) {
    TM_ATTN_CASE(1)
    TM_ATTN_CASE(2)
    TM_ATTN_CASE(3)
    TM_ATTN_CASE(4)
    TM_ATTN_CASE(5)
    TM_ATTN_CASE(6)
    TM_ATTN_CASE(7)
    TM_ATTN_CASE(8)
    default:
      return TM_ERR_UNSUPPORTED_SHAPE;
  }
#undef TM_ATTN_CASE
  return launch_status();
}

}  // namespace tmk

// q, out: [T, nh, D]; kcache, vcache: [pages, page_size, nkv, D]; block_table: [S, bt_stride] int;
// cu_q: [S + 1]; kv_before: [S]; tile_seq, tile_row0: [n_tiles]. split_keys == 0: results go to `out`.
// split_keys > 0 (a multiple of 32): partials go to part_acc [T*nh, max_splits, D] and
// part_ml [T*nh, max_splits, 2]; call tm_attention_combine afterwards.
extern "C" int tm_paged_attention(int dtype, const void* q, const void* kcache, const void* vcache,
                                  const int* block_table, int bt_stride, const int* cu_q, const int* kv_before,
                                  const int* tile_seq, const int* tile_row0, int n_tiles, void* out,
                                  float* part_acc, float* part_ml, int nh, int nkv, int D, int page_size,
                                  float scale, int window, int split_keys, int max_splits, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (D % 16 || D > 256 || D <= 0 || nkv <= 0 || nh % nkv || page_size <= 0) return TM_ERR_UNSUPPORTED_SHAPE;
  if (split_keys < 0 || split_keys % tmk::kKeyTile) return TM_ERR_UNSUPPORTED_SHAPE;
  if (split_keys > 0 && (!part_acc || !part_ml || max_splits <= 0)) return TM_ERR_SCRATCH_TOO_SMALL;
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_paged_attention<float>(q, kcache, vcache, block_table, bt_stride, cu_q, kv_before, tile_seq,
                                             tile_row0, n_tiles, out, part_acc, part_ml, nh, nkv, D, page_size,
                                             scale, window, split_keys, max_splits, stream);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_paged_attention<__nv_bfloat16>(q, kcache, vcache, block_table, bt_stride, cu_q, kv_before,
                                                     tile_seq, tile_row0, n_tiles, out, part_acc, part_ml, nh, nkv,
                                                     D, page_size, scale, window, split_keys, max_splits, stream);
  return TM_ERR_BAD_DTYPE;
}

extern "C" int tm_attention_combine(int dtype, const float* part_acc, const float* part_ml, const int* cu_q,
                                    const int* kv_before, const int* seq_of_token, void* out, int n_tokens, int nh,
                                    int D, int window, int split_keys, int max_splits, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (split_keys <= 0) return TM_ERR_UNSUPPORTED_SHAPE;
  const int rows = n_tokens * nh;
  const int warps = 4;
  const dim3 grid((rows + warps - 1) / warps);
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_pdl(tmk::attention_combine_kernel<float>, grid, dim3(warps * 32), 0, stream, part_acc, part_ml,
                           cu_q, kv_before, seq_of_token, (float*)out, n_tokens, nh, D, window, split_keys,
                           max_splits);
  else if (dtype == TM_DTYPE_BF16)
    return tmk::launch_pdl(tmk::attention_combine_kernel<__nv_bfloat16>, grid, dim3(warps * 32), 0, stream, part_acc,
                           part_ml, cu_q, kv_before, seq_of_token, (__nv_bfloat16*)out, n_tokens, nh, D, window,
                           split_keys, max_splits);
  else
    return TM_ERR_BAD_DTYPE;
  return tmk::launch_status();
}
