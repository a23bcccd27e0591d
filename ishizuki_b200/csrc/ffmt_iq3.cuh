// GGUF IQ3_XXS and IQ3_S for the warp-level kernel (mma.sync fragments).
//
// Block layouts (reference: Sources/IshizukiKit/Core/GGMLDequant.swift:313-374):
//   IQ3_XXS (98 bytes per 256 weights): d f16 @0, 64 index bytes @2 (each: four magnitudes out of a
//     256-entry grid), eight words @66: four 7-bit sign indices (eighth sign = parity) and the
//     four-bit scale s of 32 weights; w = d * (2 s + 1) / 4 * magnitude * sign.
//   IQ3_S (110 bytes): d @0, 64 index bytes @2, qh @66 (a ninth index bit each; 512-entry grid), 32
//     sign bytes @74 (all eight signs), scale nibbles @106 (per 32 weights); w = d * (2 s + 1) *
//     magnitude * sign.
//
// The decoder is the one of IQ2_XS with two lookups per eight weights: the grid lives in shared
// memory as fp16 (an entry = four magnitudes = 8 bytes = two A registers), in sixteen copies, copy
// c of entry i at i * 128 + c * 8: an 8-byte load is served sixteen lanes at a time, lane l reads
// copy l % 16. A register takes its scale by a half2 multiply with 2 s + 1 (magnitude * (2 s + 1)
// <= 1922, an exact fp16 integer) and its two signs by an integer multiply that moves its sign
// bits to bits 15 and 31, xor-ed in. Fragment mapping and activations as for IQ2_XS: a lane owns
// the sub-blocks (sixteen weights = four index bytes = two sign bytes) 4 j + t, j = 0..3, of rows
// g and g + 8.
//
// Tile (16 rows x 256 k, 1824 bytes): [2][lane][16 bytes] = for j = 2p, 2p + 1: the four index
// bytes of sub-block 4j + t of row g, then of row g + 8; [lane][16 bytes]: per j the two sign
// bytes (parity filled in) of row g, then of row g + 8; [lane][8 bytes]: per j a byte (scale |
// ninth index bits << 4) of row g, then four of row g + 8; d of rows (g, g + 8) side by side.
// (IQ3_XXS: 1568 bytes of blocks, its sign indices and scales are stored unpacked; IQ3_S: 1760.)
#pragma once
#include "ffmt_iq2xs.cuh"

namespace ishi {

// TYPE: the GGML type number, 18 IQ3_XXS, 21 IQ3_S
template <int TYPE>
struct FragIQ3 {
  static_assert(TYPE == 18 || TYPE == 21, "IQ3_XXS or IQ3_S");
  static constexpr bool kNine = TYPE == 21;  // nine index bits, explicit signs
  static constexpr int kBlock = kNine ? 110 : 98;
  static constexpr int kEntries = kNine ? 512 : 256;
  static constexpr int kSigns = 1024, kScales = 1536, kD = 1792;
  static constexpr int kTileBytes = kD + 32;
  static constexpr int kXBytes = 8 * 512;  // per unit: eight rows of 512 bytes
  static constexpr int kGrid = 8 * 16;     // first in the extra region: the rows' 16-byte skews
  static constexpr int kExtraBytes = kGrid + kEntries * 128;  // then the grid as fp16, sixteen copies interleaved
  static constexpr bool kRowMode = false;  // one activation row runs through the MMA path as well

  static __device__ __forceinline__ const uint8_t *block(const FragSrc &s, long long row, int u) {
    long long local;
    const int seg = frag_segment(s, row, &local);
    return s.w[seg] + local * s.w_row_bytes + (long long)u * kBlock;
  }

  static __device__ __forceinline__ uint8_t tile_byte(const FragSrc &s, long long p, int u, int b) {
    if (b < kSigns) {
      const int pc = b >> 9, lane = (b & 511) >> 4, i = b & 15;
      const int g = lane >> 2, t = lane & 3, slot = i >> 2, bi = i & 3;
      const long long row = p * kFragRows + g + 8 * (slot & 1);
      if (row >= s.N) return 0;
      const int sb = 4 * (2 * pc + (slot >> 1)) + t;
      return block(s, row, u)[2 + 4 * sb + bi];
    }
    if (b < kScales) {
      const int idx = b - kSigns, lane = idx >> 4, i = idx & 15;
      const int g = lane >> 2, t = lane & 3;
      const long long row = p * kFragRows + g + 8 * ((i >> 1) & 1);
      if (row >= s.N) return 0;
      const uint8_t *blk = block(s, row, u);
      const int E = 2 * (4 * (i >> 2) + t) + (i & 1);  // entry (eight weights) of the block
      if (kNine) return blk[74 + E];
      const uint8_t *aux = blk + 66 + 4 * (E >> 2);
      const uint32_t word = (uint32_t)aux[0] | ((uint32_t)aux[1] << 8) | ((uint32_t)aux[2] << 16) | ((uint32_t)aux[3] << 24);
      const uint32_t s7 = (word >> (7 * (E & 3))) & 127u;
      return (uint8_t)(s7 | ((uint32_t)(__popc(s7) & 1) << 7));
    }
    if (b < kD) {
      const int idx = b - kScales, lane = idx >> 3, i = idx & 7;
      const int g = lane >> 2, t = lane & 3;
      const long long row = p * kFragRows + g + 8 * (i >> 2);
      if (row >= s.N) return 0;
      const uint8_t *blk = block(s, row, u);
      const int sb = 4 * (i & 3) + t;
      if (kNine) {
        const uint32_t scale = ((uint32_t)blk[106 + (sb >> 2)] >> (4 * ((sb >> 1) & 1))) & 15u;
        const uint32_t high = ((uint32_t)blk[66 + (sb >> 1)] >> (4 * (sb & 1))) & 15u;  // a bit per index byte
        return (uint8_t)(scale | (high << 4));
      }
      return (uint8_t)(blk[66 + 4 * (sb >> 1) + 3] >> 4);
    }
    const int idx = b - kD;
    const long long row = p * kFragRows + (idx >> 2) + 8 * ((idx >> 1) & 1);
    if (row >= s.N) return 0;
    return block(s, row, u)[idx & 1];
  }

  static __device__ __forceinline__ uint16_t tile_halfword(const FragSrc &s, long long p, int u, int hw) {
    return (uint16_t)(tile_byte(s, p, u, 2 * hw) | ((uint32_t)tile_byte(s, p, u, 2 * hw + 1) << 8));
  }

  static __device__ __forceinline__ uint32_t row_stride(const FragArgs &a) { return (uint32_t)a.umax * 512u + 16u; }

  // the grid, set up ahead of the dependency wait; sixteen consecutive threads store the sixteen
  // copies of an entry, 128 contiguous bytes
  static __device__ __forceinline__ void before_wait(const FragArgs &a, uint32_t xfrag) {
    const uint32_t grid = xfrag + (uint32_t)a.umax * kXBytes + kGrid;
    for (int i = threadIdx.x; i < kEntries * 16; i += blockDim.x) {
      const uint32_t bytes = kNine ? d_iq3s_grid[i >> 4] : d_iq3xxs_grid[i >> 4];  // four magnitudes, a byte each
      const __half2 lo = __halves2half2(__int2half_rn((int)(bytes & 0xffu)), __int2half_rn((int)((bytes >> 8) & 0xffu)));
      const __half2 hi = __halves2half2(__int2half_rn((int)((bytes >> 16) & 0xffu)), __int2half_rn((int)(bytes >> 24)));
      sts64(grid + (uint32_t)i * 8u, *reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
    }
  }

  // the activations as for IQ2_XS: the rows as they lie in x
  template <class F>
  static __device__ __forceinline__ void stage_x(const FragArgs &a, uint32_t xfrag, int ub0, int uc, F &&after_loads) {
    FragIQ2<17>::stage_x(a, xfrag, ub0, uc, after_loads);
  }

  // eight weights as four A registers, magnitude * (2 s + 1) * sign: the two grid indices (this
  // lane's copy of the grid), the eight sign bits
  static __device__ __forceinline__ void entry(uint32_t (&r)[4], uint32_t ia, uint32_t ib, uint32_t s8, uint32_t grid, __half2 scale) {
    const uint2 ma = lds64(grid + ia * 128u), mb = lds64(grid + ib * 128u);
    const uint32_t mag[4] = {ma.x, ma.y, mb.x, mb.y};
    // sign bits 2r and 2r + 1 to bits 15 and 31
    const uint32_t mul[4] = {0x40008000u, 0x10002000u, 0x04000800u, 0x01000200u};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 v = __hmul2(*reinterpret_cast<const __half2 *>(&mag[i]), scale);
      r[i] = *reinterpret_cast<const uint32_t *>(&v) ^ ((s8 * mul[i]) & 0x80008000u);
    }
  }
  // index byte i of word q, with its ninth bit from bit 4 + i of the sub-block's byte
  static __device__ __forceinline__ uint32_t index_of(uint32_t q, uint32_t byte, int i) {
    const uint32_t low = (q >> (8 * i)) & 0xffu;
    return kNine ? low | ((byte << (4 - i)) & 0x100u) : low;
  }

  // One tile against the activations of its unit; acc is the warp's C fragment.
  template <int MODE>
  static __device__ __forceinline__ void unit(float (&acc)[4], const FragArgs &a, uint32_t tile, uint32_t xbase, int uq,
                                              int g, int t, int lane) {
    const uint32_t R = row_stride(a);
    const uint32_t grid = xbase + (uint32_t)a.umax * kXBytes + kGrid + (uint32_t)(lane & 15) * 8u;
    const uint32_t xrow = xbase + (uint32_t)g * R + (uint32_t)uq * 512u + (uint32_t)t * 32u;
    const uint4 sg = lds128(tile + kSigns + (uint32_t)lane * 16u);  // word j: sign bytes of row g (low half), of row g + 8
    const uint2 sw = lds64(tile + kScales + (uint32_t)lane * 8u);   // byte j: scale | ninth bits << 4; row g, row g + 8
    const uint32_t sgw[4] = {sg.x, sg.y, sg.z, sg.w};
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int pc = 0; pc < 2; ++pc) {
      const uint4 w = lds128(tile + (uint32_t)pc * 512u + (uint32_t)lane * 16u);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = 2 * pc + e;
        const uint32_t q0 = e ? w.z : w.x, q1 = e ? w.w : w.y;  // the sub-block's four index bytes of row g, of row g + 8
        const uint32_t y0 = sw.x >> (8 * j), y1 = sw.y >> (8 * j);
        const __half2 s0 = FragIQ2<17>::scale_of(y0, 0), s1 = FragIQ2<17>::scale_of(y1, 0);
        uint32_t lo0[4], hi0[4], lo1[4], hi1[4];
        entry(lo0, index_of(q0, y0, 0), index_of(q0, y0, 1), sgw[j] & 0xffu, grid, s0);
        entry(hi0, index_of(q0, y0, 2), index_of(q0, y0, 3), (sgw[j] >> 8) & 0xffu, grid, s0);
        entry(lo1, index_of(q1, y1, 0), index_of(q1, y1, 1), (sgw[j] >> 16) & 0xffu, grid, s1);
        entry(hi1, index_of(q1, y1, 2), index_of(q1, y1, 3), sgw[j] >> 24, grid, s1);
        const uint4 b0 = lds128(xrow + (uint32_t)j * 128u), b1 = lds128(xrow + (uint32_t)j * 128u + 16u);
        if (j == 0)
          mma16816_first(c, lo0[0], lo1[0], lo0[1], lo1[1], b0.x, b0.y);
        else
          mma16816(c, lo0[0], lo1[0], lo0[1], lo1[1], b0.x, b0.y);
        mma16816(c, lo0[2], lo1[2], lo0[3], lo1[3], b0.z, b0.w);
        mma16816(c, hi0[0], hi1[0], hi0[1], hi1[1], b1.x, b1.y);
        mma16816(c, hi0[2], hi1[2], hi0[3], hi1[3], b1.z, b1.w);
      }
    }
    const uint32_t dd = lds32(tile + (uint32_t)kD + (uint32_t)g * 4u);
    const float f = kNine ? 1.0f : 0.25f;
    const float d0 = half_bits_to_float(dd & 0xffffu) * f, d1 = half_bits_to_float(dd >> 16) * f;
    acc[0] = fmaf(d0, c[0], acc[0]);
    acc[1] = fmaf(d0, c[1], acc[1]);
    acc[2] = fmaf(d1, c[2], acc[2]);
    acc[3] = fmaf(d1, c[3], acc[3]);
  }
};

}  // namespace ishi
