// The body of split-key decode attention for one (request, kv head, key split): 4 warps, 128 threads.
// See attention_decode_bf16.cu for the method. Returns false when the unit has no keys.
//
// `wait_for_step` is called once, before the unit touches anything the kernel in front of it on the stream
// wrote: the queries, and the keys and values of the step's own tokens (positions >= `before`). Keys and
// values of older positions were written by earlier steps, so their copies are asked for BEFORE that call:
// launched with programmatic dependent launch, the kernel gets its table lookups and most of its data on
// the way while the kernel in front of it is still running.
#pragma once

#include "mma_util.cuh"

namespace tmk {

constexpr int kDecBN = 64;       // keys per stage
constexpr int kDecWarps = 4;

// Bytes of shared memory one unit needs: two stages of K and V tiles, reused for the 4 warps' merge.
template <int D> constexpr int decode_unit_smem_bytes() {
  return (2 * 2 * kDecBN * D * 2) > (kDecWarps * 16 * (D + 2) * 4) ? (2 * 2 * kDecBN * D * 2)
                                                                     : (kDecWarps * 16 * (D + 2) * 4);
}

template <int D, typename Sync, typename Wait>
__device__ __forceinline__ bool decode_attention_unit(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kcache,
    const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ table, int q_start, int q_len, int before,
    int kvh, int z, float* __restrict__ part_acc, float* __restrict__ part_ml, int nh, int nkv, int page_size,
    float scale_log2, int window, int split_keys, int max_splits, unsigned char* smem, int tid, Sync sync,
    Wait wait_for_step) {
  constexpr int CH = D / 8;                 // 16-byte chunks per row
  constexpr int KS = D / 16;                // k-steps of the score product
  constexpr int NT = D / 8;                 // 8-wide output tiles
  constexpr int TILE_BYTES = kDecBN * D * 2;
  // [stage][K | V] tiles; after the loop the same memory holds the 4 warps' states for the merge.
  const uint32_t smem_base = smem_u32(smem);
  const int G = nh / nkv;
  const int n_rows = min(q_len * G, 16);
  if (n_rows <= 0) return false;
  const int p_min = before, p_max = before + (n_rows - 1) / G;
  int j_lo = window > 0 ? max(0, p_min - window + 1) : 0;
  int j_hi = p_max;
  j_lo = max(j_lo, z * split_keys);
  j_hi = min(j_hi, (z + 1) * split_keys - 1);
  if (j_lo > j_hi) return false;

  const int lane = tid & 31, warp = tid >> 5;
  const int r0 = lane >> 2, r1 = r0 + 8;    // the two tile rows this thread's accumulators belong to
  const int cpair = (lane & 3) * 2;

  uint32_t qa[KS][4];
  const int p_r0 = r0 < n_rows ? before + r0 / G : -1, p_r1 = r1 < n_rows ? before + r1 / G : -1;
  const int lo_r0 = window > 0 ? max(0, p_r0 - window + 1) : 0, lo_r1 = window > 0 ? max(0, p_r1 - window + 1) : 0;

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // running max (log2 units) and sum per row
  float o[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;

  const int kb_first = (j_lo / kDecBN) * kDecBN;
  const int n_blocks = (j_hi - kb_first) / kDecBN + 1;

  auto load_block = [&](int stage, int kb) {
    const uint32_t k_dst = smem_base + stage * 2 * TILE_BYTES, v_dst = k_dst + TILE_BYTES;
    for (int idx = tid; idx < kDecBN * CH; idx += kDecWarps * 32) {
      const int row = idx / CH, c = idx - row * CH;
      const int j = kb + row;
      const bool ok = j >= j_lo && j <= j_hi;
      size_t src = 0;
      if (ok) {
        const int page = table[j / page_size];
        src = (((size_t)page * page_size + (j % page_size)) * nkv + kvh) * D + c * 8;
      }
      const uint32_t off = row * (D * 2) + ((c ^ (row & 7)) << 4);
      cp_async16(k_dst + off, kcache + src, ok);
      cp_async16(v_dst + off, vcache + src, ok);
    }
  };

  // Block k of the unit into stage k & 1. A block that holds keys of the step's own tokens has to wait for the
  // kernel that wrote them; all the others are asked for at once.
  bool waited = false;
  auto issue = [&](int k) {
    const int kb = kb_first + k * kDecBN;
    if (!waited && kb + kDecBN > before) {
      wait_for_step();
      waited = true;
    }
    load_block(k & 1, kb);
    cp_async_commit();
  };
  issue(0);
  if (n_blocks > 1) issue(1);
  if (!waited) {
    wait_for_step();
    waited = true;
  }
  // Query fragments straight from global memory (rows beyond n_rows are zero).
  {
    const __nv_bfloat16* qr0 = nullptr;
    const __nv_bfloat16* qr1 = nullptr;
    if (r0 < n_rows) qr0 = q + ((size_t)(q_start + r0 / G) * nh + kvh * G + r0 % G) * D;
    if (r1 < n_rows) qr1 = q + ((size_t)(q_start + r1 / G) * nh + kvh * G + r1 % G) * D;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int c = ks * 16 + cpair;
      qa[ks][0] = qr0 ? __ldcg(reinterpret_cast<const unsigned int*>(qr0 + c)) : 0u;
      qa[ks][1] = qr1 ? __ldcg(reinterpret_cast<const unsigned int*>(qr1 + c)) : 0u;
      qa[ks][2] = qr0 ? __ldcg(reinterpret_cast<const unsigned int*>(qr0 + c + 8)) : 0u;
      qa[ks][3] = qr1 ? __ldcg(reinterpret_cast<const unsigned int*>(qr1 + c + 8)) : 0u;
    }
  }
  for (int b = 0; b < n_blocks; ++b) {
    const int kb = kb_first + b * kDecBN;
    const int stage = b & 1;
    if (b >= 1 && b + 1 < n_blocks) issue(b + 1);      // (its stage was given back at the end of the last trip)
    if (b + 1 < n_blocks) {
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    sync();

    const int kr = warp * 16;                // this warp's 16 keys of the block
    if (kb + kr <= j_hi && kb + kr + 15 >= j_lo) {
      const uint32_t k_base = smem_base + stage * 2 * TILE_BYTES, v_base = k_base + TILE_BYTES;
      float sc[2][4];
#pragma unroll
      for (int t = 0; t < 2; ++t) sc[t][0] = sc[t][1] = sc[t][2] = sc[t][3] = 0.f;
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
      // Mask, scale into log2 units, online softmax over this warp's 16 keys.
      float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = kb + kr + t * 8 + cpair + e;
          const bool in = j >= j_lo && j <= j_hi;
          sc[t][e] = (in && j <= p_r0 && j >= lo_r0) ? sc[t][e] * scale_log2 : -INFINITY;
          sc[t][2 + e] = (in && j <= p_r1 && j >= lo_r1) ? sc[t][2 + e] * scale_log2 : -INFINITY;
          tmax0 = fmaxf(tmax0, sc[t][e]);
          tmax1 = fmaxf(tmax1, sc[t][2 + e]);
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
        for (int t = 0; t < 2; ++t)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            p[t][e] = mn0 == -INFINITY ? 0.f : exp2f(sc[t][e] - mn0);
            p[t][2 + e] = mn1 == -INFINITY ? 0.f : exp2f(sc[t][2 + e] - mn1);
            ps0 += p[t][e];
            ps1 += p[t][2 + e];
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
      for (int t = 0; t < NT; ++t) {
        o[t][0] *= corr0;
        o[t][1] *= corr0;
        o[t][2] *= corr1;
        o[t][3] *= corr1;
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
    sync();   // the stage may be refilled by the next trip's loads
  }

  // Merge the 4 warps' states in warp order: smem holds [warp][16 rows][D] acc, then [warp][16][2] (m, l).
  float* macc = reinterpret_cast<float*>(smem);
  float* mml = macc + kDecWarps * 16 * D;
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    const int c = t * 8 + cpair;
    *reinterpret_cast<float2*>(macc + (warp * 16 + r0) * D + c) = make_float2(o[t][0], o[t][1]);
    *reinterpret_cast<float2*>(macc + (warp * 16 + r1) * D + c) = make_float2(o[t][2], o[t][3]);
  }
  if ((lane & 3) == 0) {
    mml[(warp * 16 + r0) * 2] = m0;
    mml[(warp * 16 + r0) * 2 + 1] = l0;
    mml[(warp * 16 + r1) * 2] = m1;
    mml[(warp * 16 + r1) * 2 + 1] = l1;
  }
  sync();
  constexpr float kLn2 = 0.6931471805599453f;
  for (int idx = tid; idx < n_rows * D; idx += kDecWarps * 32) {
    const int r = idx / D, d = idx - r * D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) mx = fmaxf(mx, mml[(w * 16 + r) * 2]);
    float acc = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float mw = mml[(w * 16 + r) * 2];
      const float wgt = mw == -INFINITY ? 0.f : exp2f(mw - mx);
      acc = fmaf(macc[(w * 16 + r) * D + d], wgt, acc);
      lsum = fmaf(mml[(w * 16 + r) * 2 + 1], wgt, lsum);
    }
    const size_t orow = (size_t)(q_start + r / G) * nh + kvh * G + r % G;
    part_acc[(orow * max_splits + z) * D + d] = acc;
    if (d == 0) {
      part_ml[(orow * max_splits + z) * 2] = mx * kLn2;     // natural-log units, as the combine kernel reads
      part_ml[(orow * max_splits + z) * 2 + 1] = lsum;
    }
  }
  return true;
}

}  // namespace tmk
