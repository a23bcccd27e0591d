// GGUF IQ4_XS for the warp-level kernel (mma.sync fragments).
//
// Block layout (136 bytes per 256 weights; reference: Sources/IshizukiKit/Core/GGMLDequant.swift:222-241):
//   d f16 @0, scales_h u16 @2, scales_l[4] @4, qs[128] @8. Sub-block ib (32 weights) has the six-bit
//   scale ls = (scales_l[ib / 2] >> 4 (ib % 2)) & 15 | ((scales_h >> 2 ib) & 3) << 4 and sixteen
//   bytes qs[16 ib + j]: weight j takes the low nibble, weight j + 16 the high nibble, as indices
//   into the sixteen non-uniform values kvalues_iq4nl; w = d * (ls - 32) * value.
//
// A byte is two weights, 16 apart: exactly one A register (an fp16 pair), looked up whole in a
// 256-entry table of value pairs in shared memory (one copy per lane, so that the 32 lookups of a
// warp never meet in a bank). The k order inside the MMA follows the bytes: in k-step s (0, 1) of
// sub-block ib the lane t uses bytes 4t + 2s and 4t + 2s + 1 of the sub-block, i.e. the MMA's k
// columns (2t, 2t + 1) are the weights (4t + 2s, 4t + 2s + 16) and (2t + 8, 2t + 9) the weights
// (4t + 2s + 1, 4t + 2s + 17); the activations are staged in the same order. A lane thus owns the
// 32-bit word t of every sub-block of its two rows. The table values are small integers, exact in
// fp16; a sub-block's two k-steps accumulate in fp32 inside the MMA and take the integer ls - 32
// afterwards, the block's d at the end of the tile.
//
// Tile (16 rows x 256 k, 2208 bytes): words [4][lane][row g: sub-blocks 2j, 2j + 1; row g + 8: the
// same] @0, per row the eight scales ls as bytes @2048, d of rows (g, g + 8) side by side @2176.
#pragma once
#include "ggml_decode.cuh"
#include "ishi_fragstream.cuh"

namespace ishi {

struct FragIQ4XS {
  static constexpr int kTileBytes = 2048 + 128 + 32;
  static constexpr int kXBytes = 4096;                // per unit: sixteen k-steps of 256 bytes
  static constexpr int kExtraBytes = 256 * 128;       // the pair table: entry e of lane l's copy at e * 128 + l * 4
  static constexpr bool kRowMode = false;             // one activation row runs through the MMA path as well

  static __device__ __forceinline__ const uint8_t *block(const FragSrc &s, long long row, int u) {
    long long local;
    const int seg = frag_segment(s, row, &local);
    return s.w[seg] + local * s.w_row_bytes + (long long)u * 136;
  }

  static __device__ __forceinline__ uint8_t tile_byte(const FragSrc &s, long long p, int u, int b) {
    if (b < 2048) {
      const int j = b >> 9, lane = (b & 511) >> 4, i = b & 15;
      const int g = lane >> 2, t = lane & 3, wi = i >> 2, bi = i & 3;
      const long long row = p * kFragRows + g + 8 * (wi >> 1);
      if (row >= s.N) return 0;
      const int sb = 2 * j + (wi & 1);
      return block(s, row, u)[8 + 16 * sb + 4 * t + bi];
    }
    if (b < 2176) {
      const int idx = b - 2048, sb = idx & 7;
      const long long row = p * kFragRows + (idx >> 3);
      if (row >= s.N) return 32;  // d = 0 there as well
      const uint8_t *blk = block(s, row, u);
      const uint32_t low = (blk[4 + sb / 2] >> (4 * (sb % 2))) & 0xfu;
      const uint32_t high = (((uint32_t)blk[2] | ((uint32_t)blk[3] << 8)) >> (2 * sb)) & 3u;
      return (uint8_t)(low | (high << 4));
    }
    const int idx = b - 2176;
    const long long row = p * kFragRows + (idx >> 2) + 8 * ((idx >> 1) & 1);
    if (row >= s.N) return 0;
    return block(s, row, u)[idx & 1];
  }

  static __device__ __forceinline__ uint16_t tile_halfword(const FragSrc &s, long long p, int u, int hw) {
    return (uint16_t)(tile_byte(s, p, u, 2 * hw) | ((uint32_t)tile_byte(s, p, u, 2 * hw + 1) << 8));
  }

  // the pair table, filled ahead of the dependency wait: it depends on no earlier launch
  static __device__ __forceinline__ void before_wait(const FragArgs &a, uint32_t xfrag) {
    const uint32_t table = xfrag + (uint32_t)a.umax * kXBytes;
    for (int i = threadIdx.x; i < 256 * 32; i += blockDim.x) {
      const int e = i >> 5;  // consecutive threads store one entry's 32 copies: consecutive banks
      const __half2 pair = __halves2half2(__int2half_rn((int)d_kvalues_iq4nl[e & 15]), __int2half_rn((int)d_kvalues_iq4nl[e >> 4]));
      sts32(table + (uint32_t)i * 4u, *reinterpret_cast<const uint32_t *>(&pair));
    }
  }

  // Activations of the CTA's column range into fragment order. A warp task is (unit, activation
  // row r): lane l loads k = 8l .. 8l + 7, a quarter of sub-block l / 4: the low-nibble weights
  // 8 (l % 4) ... + 7 when l % 4 < 2, else the high-nibble weights 16 + 8 (l % 4 - 2) ... + 7. Lanes
  // l and l ^ 2 hold the two halves of the same eight pairs: they swap four values each, the first
  // builds the pairs of t = 2 (l % 4), the second those of t + 1. The B registers of k-step
  // ks = 2 ib + s and quad row r lie at ks * 256 + ((r ^ (ks % 8)) * 4 + t) * 8; the xor spreads the
  // stores over the banks, a warp's read of one k-step is still one 256-byte run.
  // after_loads() runs once, when the first loads are in flight. No rotation here.
  template <class F>
  static __device__ __forceinline__ void stage_x(const FragArgs &a, uint32_t xfrag, int ub0, int uc, F &&after_loads) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int tasks = uc * 8;
    constexpr int kBatch = 8;
    const __half *xl = a.x + (long long)ub0 * 256 + lane * 8;
    const int ib = lane >> 2, r4 = lane & 3;
    const bool second = r4 >= 2;
    const int t = second ? 2 * (r4 - 2) + 1 : 2 * r4;
    if (warp >= tasks) after_loads();  // a warp without a task
    for (int i0 = warp; i0 < tasks; i0 += nw * kBatch) {
      uint4 v[kBatch];
#pragma unroll
      for (int e = 0; e < kBatch; ++e) {
        const int i = i0 + e * nw;
        v[e] = make_uint4(0u, 0u, 0u, 0u);
        if (i < tasks && (i & 7) < a.M)
          v[e] = __ldg(reinterpret_cast<const uint4 *>(xl + (long long)(i & 7) * a.K + (i >> 3) * 256));
      }
      if (i0 == warp) after_loads();
#pragma unroll
      for (int e = 0; e < kBatch; ++e) {
        const int i = i0 + e * nw;
        if (i >= tasks) break;
        const int r = i & 7;
        const uint32_t base = xfrag + (uint32_t)(i >> 3) * kXBytes;
        const uint32_t got0 = __shfl_xor_sync(0xffffffffu, second ? v[e].x : v[e].z, 2);
        const uint32_t got1 = __shfl_xor_sync(0xffffffffu, second ? v[e].y : v[e].w, 2);
        const uint32_t lo0 = second ? got0 : v[e].x, lo1 = second ? got1 : v[e].y;
        const uint32_t hi0 = second ? v[e].z : got0, hi1 = second ? v[e].w : got1;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const int ks = 2 * ib + s;
          const uint32_t lo = s ? lo1 : lo0, hi = s ? hi1 : hi0;
          sts64(base + (uint32_t)ks * 256u + (uint32_t)(((r ^ (ks & 7)) * 4 + t) * 8), prmt(lo, hi, 0x5410u), prmt(lo, hi, 0x7632u));
        }
      }
    }
  }

  // the value pair of byte `byte` of word w
  static __device__ __forceinline__ uint32_t pair_of(uint32_t w, int byte, uint32_t table) {
    return lds32(prmt(w, 0u, 0x4440u | (uint32_t)byte) * 128u + table);
  }
  // 8388608 + byte `byte` of word w, as a float
  static __device__ __forceinline__ float byte_float(uint32_t w, int byte) {
    return __uint_as_float(prmt(w, 0x4b000000u, 0x7440u | (uint32_t)byte));
  }

  // One tile against the activations of its unit; acc is the warp's C fragment.
  template <int MODE>
  static __device__ __forceinline__ void unit(float (&acc)[4], const FragArgs &a, uint32_t tile, uint32_t xbase, int uq,
                                              int g, int t, int lane) {
    const uint32_t xu = xbase + (uint32_t)uq * kXBytes;
    const uint32_t table = xbase + (uint32_t)a.umax * kXBytes + (uint32_t)lane * 4u;
    const uint2 sc0 = lds64(tile + 2048u + (uint32_t)g * 8u), sc1 = lds64(tile + 2048u + (uint32_t)(g + 8) * 8u);
    float su[4] = {0.f, 0.f, 0.f, 0.f};  // sum over the sub-blocks of (ls - 32) * (sum of value * x), d follows at the end
    const uint32_t xl = xu + (uint32_t)t * 8u;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 q = lds128(tile + (uint32_t)j * 512u + (uint32_t)lane * 16u);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int sb = 2 * j + e;
        const uint32_t w0 = e ? q.y : q.x, w1 = e ? q.w : q.z;
        float part[4];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const int ks = 2 * sb + s;
          const uint2 b = lds64(xl + (uint32_t)ks * 256u + (uint32_t)((g ^ (ks & 7)) * 32));
          const uint32_t a0 = pair_of(w0, 2 * s, table), a2 = pair_of(w0, 2 * s + 1, table);
          const uint32_t a1 = pair_of(w1, 2 * s, table), a3 = pair_of(w1, 2 * s + 1, table);
          if (s == 0) mma16816_first(part, a0, a1, a2, a3, b.x, b.y);
          else mma16816(part, a0, a1, a2, a3, b.x, b.y);
        }
        const float f0 = byte_float(sb < 4 ? sc0.x : sc0.y, sb & 3) - 8388640.f;  // ls - 32, exact
        const float f1 = byte_float(sb < 4 ? sc1.x : sc1.y, sb & 3) - 8388640.f;
        su[0] = fmaf(f0, part[0], su[0]), su[1] = fmaf(f0, part[1], su[1]);
        su[2] = fmaf(f1, part[2], su[2]), su[3] = fmaf(f1, part[3], su[3]);
      }
    }
    const uint32_t dd = lds32(tile + 2176u + (uint32_t)g * 4u);
    const float d0 = half_bits_to_float(dd & 0xffffu), d1 = half_bits_to_float(dd >> 16);
    acc[0] = fmaf(d0, su[0], acc[0]), acc[1] = fmaf(d0, su[1], acc[1]);
    acc[2] = fmaf(d1, su[2], acc[2]), acc[3] = fmaf(d1, su[3], acc[3]);
  }
};

}  // namespace ishi
