// Merging the key chunks of one (row tile, kv head) of prompt attention: the partial sums, maxima and
// denominators that the chunks' blocks left are combined in chunk order, each weighted by 2^(its maximum - the
// maximum so far), and the normalised rows are written as bfloat16. Used by the block that finishes a tile last.
#pragma once

#include <cuda_bf16.h>

#include "mma_util.cuh"

namespace tmk {

// part_acc [slots * nkv, TILE_ROWS, D] and part_ml [slots * nkv, TILE_ROWS, 2] (maximum in log2 units,
// denominator); the tile's chunks lie in slots slot0 .. slot0 + n_chunks - 1. Row r of the tile is (token,
// head) row row0 + r of the request, whose first token is row q_start of `out` [tokens, nh, D]. Rows a chunk
// had no key for carry a maximum of -inf and a zero denominator and drop out. Each thread works on ITEMS
// 4-float pieces at once: one piece and chunk at a time, with each weight waiting for the one before, the
// merge took longer than the unit's products.
template <int D, int TILE_ROWS, int THREADS, int ITEMS>
__device__ __forceinline__ void merge_tile_chunks(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                                  int slot0, int n_chunks, int nkv, int kvh, int n_rows, int row0,
                                                  int G, int q_start, int nh, __nv_bfloat16* __restrict__ out, int tid) {
  constexpr int PIECES = D / 4;
  const int total = n_rows * PIECES;
  for (int base = tid; base < total; base += THREADS * ITEMS) {
    bool has[ITEMS];
    int r[ITEMS], d[ITEMS];
    float mx[ITEMS], lsum[ITEMS], acc[ITEMS][4];
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const int idx = base + k * THREADS;
      has[k] = idx < total;
      r[k] = has[k] ? idx / PIECES : 0;
      d[k] = has[k] ? (idx - r[k] * PIECES) * 4 : 0;
      mx[k] = -INFINITY;
      lsum[k] = 0.f;
      acc[k][0] = acc[k][1] = acc[k][2] = acc[k][3] = 0.f;
    }
    // First each row's maximum over the chunks, then every chunk weighted by 2^(its maximum - that): the
    // weights do not depend on one another, so nothing waits for an exponential before it.
#pragma unroll 4
    for (int c = 0; c < n_chunks; ++c)
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const size_t prow = ((size_t)(slot0 + c) * nkv + kvh) * TILE_ROWS + r[k];
        mx[k] = fmaxf(mx[k], __ldcg(part_ml + prow * 2));
      }
#pragma unroll 2
    for (int c = 0; c < n_chunks; ++c) {
      float2 ml[ITEMS];
      float4 pa[ITEMS];
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const size_t prow = ((size_t)(slot0 + c) * nkv + kvh) * TILE_ROWS + r[k];
        ml[k] = __ldcg(reinterpret_cast<const float2*>(part_ml + prow * 2));
        pa[k] = __ldcg(reinterpret_cast<const float4*>(part_acc + prow * D + d[k]));
      }
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const float w = ml[k].x == -INFINITY ? 0.f : exp2f(ml[k].x - mx[k]);
        lsum[k] += ml[k].y * w;
        acc[k][0] += pa[k].x * w;
        acc[k][1] += pa[k].y * w;
        acc[k][2] += pa[k].z * w;
        acc[k][3] += pa[k].w * w;
      }
    }
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      if (!has[k]) continue;
      const float inv = lsum[k] > 0.f ? 1.0f / lsum[k] : 0.f;
      const int row = row0 + r[k], tok = row / G, g = row - tok * G;
      uint2 ov;
      ov.x = pack_bf16(acc[k][0] * inv, acc[k][1] * inv);
      ov.y = pack_bf16(acc[k][2] * inv, acc[k][3] * inv);
      *reinterpret_cast<uint2*>(out + ((size_t)(q_start + tok) * nh + kvh * G + g) * D + d[k]) = ov;
    }
  }
}

}  // namespace tmk
