// GGUF IQ2_XS for the warp-level kernel (mma.sync fragments).
//
// Block layout (74 bytes per 256 weights; reference: Sources/IshizukiKit/Core/GGMLDequant.swift
// :264-285 and the kernel body at Sources/IshizukiKit/Core/GGMLKernels.swift:664-676):
//   d f16 @0, thirty-two u16 @2 (bits 0-8: index into the 512-entry grid of eight magnitudes out of
//   {8, 25, 43}; bits 9-15: index into the 128 sign patterns, whose eighth sign is the parity of
//   the seven), eight scale bytes @66 (low nibble: first sixteen weights of a 32-group, high
//   nibble: the second sixteen);  w = d * (2 s + 1) / 8 * magnitude * sign.
//
// Decode: the grid lives in shared memory as fp16 (512 entries x 16 bytes = one 16-byte load per
// eight weights = four A registers), in eight copies, copy c of entry i at i * 128 + c * 16: a
// 16-byte load is served eight lanes at a time, lane l reads copy l % 8, so the eight lanes of a
// pass always hit eight different bank groups whatever their indices are (one copy alone measured
// 2.2 million bank conflicts per launch and warps stalled on shared memory 3.7 cycles per issue); a register then takes its scale by a half2 multiply with
// 2 s + 1 (magnitude * (2 s + 1) <= 1333 is an exact fp16 integer) and its two signs by an
// integer multiply that moves sign bits 2r and 2r + 1 to bits 15 and 31, xor-ed in. With the scale
// inside the fragments a whole tile accumulates in one MMA chain; d / 8 remains for fp32.
//
// Fragment mapping (m16n8k16; lane g = lane / 4, t = lane % 4 holds weight rows g and g + 8): a
// lane owns the sub-blocks (sixteen weights = two u16 = one scale) 4 j + t, j = 0..3, of both rows.
// The eight registers of a sub-block feed four k-steps m = 0..3: slots (2t, 2t + 1) are weights
// 4m, 4m + 1 and slots (2t + 8, 2t + 9) weights 4m + 2, 4m + 3 of the sub-block, so that the
// activations are used as they lie in memory: 32 contiguous bytes of x per lane and sub-block.
//
// Tile (16 rows x 256 k, 1184 bytes = 16 * 74): [2][lane][16 bytes] = for j = 2p, 2p + 1: the two
// u16 of sub-block 4j + t of row g, then of row g + 8; then [lane][4 bytes]: the lane's four scale
// nibbles of row g (16 bits, nibble j), then of row g + 8; then d of rows (g, g + 8) side by side.
//
// Activations of a unit in shared memory: eight rows of 256 fp16 as they lie in x, the rows
// umax * 512 + 16 bytes apart (a quarter warp's 16-byte loads then sweep all banks).
//
// The same decoder serves the two sibling formats, which differ in where a block keeps the same
// three things (a grid index and eight signs per eight weights, a four-bit scale):
//   IQ2_XXS (66 bytes; GGMLDequant.swift:243-262): per 32 weights four index bytes into a 256-entry
//     grid and one word of four 7-bit sign indices and the scale of all 32. Its tile is written in
//     the IQ2_XS form (u16 = index | sign index << 9, the scale once per sixteen weights): 1184
//     bytes for 1056 of blocks, the one format here whose tiled copy is larger than its blocks.
//   IQ2_S (82 bytes; GGMLDequant.swift:287-311): index bytes, sign bytes (all eight signs, no
//     parity), two more index bits per eight weights, scales as IQ2_XS; 1024-entry grid. Tile: per
//     sub-block and row one word [index 0][index 1][signs 0][signs 1] where IQ2_XS has its two u16,
//     then [lane][8 bytes]: per sub-block j a byte (scale | high index bits << 4) of row g, then
//     of row g + 8; 1312 bytes = 16 * 82. Its grid has four copies (64 KB), two lanes of a pass
//     share one.
#pragma once
#include "ggml_decode.cuh"
#include "ishi_fragstream.cuh"
#include "iq2xs_tables.h"

namespace ishi {

static __device__ const uint16_t g_iq2xs_frag_codes[512] = {ISHI_IQ2XS_CODES_LIST};

// TYPE: the GGML type number, 17 IQ2_XS, 16 IQ2_XXS, 22 IQ2_S
template <int TYPE>
struct FragIQ2 {
  static_assert(TYPE == 17 || TYPE == 16 || TYPE == 22, "IQ2_XS, IQ2_XXS or IQ2_S");
  static constexpr bool kWide = TYPE == 22;                  // IQ2_S: ten index bits, eight explicit signs
  static constexpr int kBlock = TYPE == 17 ? 74 : TYPE == 16 ? 66 : 82;
  static constexpr int kEntries = TYPE == 17 ? 512 : TYPE == 16 ? 256 : 1024;
  static constexpr int kCopies = kWide ? 4 : 8;              // of the grid
  static constexpr int kScales = 1024;                       // offset of the per-lane scale bytes
  static constexpr int kD = kScales + (kWide ? 256 : 128);   // offset of d
  static constexpr int kTileBytes = kD + 32;
  static constexpr int kXBytes = 8 * 512;        // per unit: eight rows of 512 bytes
  static constexpr int kGrid = 8 * 16;           // first in the extra region: the rows' 16-byte skews
  static constexpr int kExtraBytes = kGrid + kEntries * kCopies * 16;  // then the grid as fp16, its copies interleaved
  static constexpr bool kRowMode = false;        // one activation row runs through the MMA path as well

  static __device__ __forceinline__ const uint8_t *block(const FragSrc &s, long long row, int u) {
    long long local;
    const int seg = frag_segment(s, row, &local);
    return s.w[seg] + local * s.w_row_bytes + (long long)u * kBlock;
  }

  // entry E (eight weights) of a block in the IQ2_XS form: grid index | sign index << 9
  static __device__ __forceinline__ uint32_t entry16(const uint8_t *blk, int E) {
    if (TYPE == 17) return (uint32_t)blk[2 + 2 * E] | ((uint32_t)blk[3 + 2 * E] << 8);
    const uint8_t *grp = blk + 2 + 8 * (E >> 2);
    const uint32_t aux2 = (uint32_t)grp[4] | ((uint32_t)grp[5] << 8) | ((uint32_t)grp[6] << 16) | ((uint32_t)grp[7] << 24);
    return (uint32_t)grp[E & 3] | (((aux2 >> (7 * (E & 3))) & 127u) << 9);
  }
  // the four-bit scale of sub-block sb (sixteen weights)
  static __device__ __forceinline__ uint32_t scale4(const uint8_t *blk, int sb) {
    if (TYPE == 16) return (uint32_t)blk[2 + 8 * (sb >> 1) + 7] >> 4;
    return ((uint32_t)blk[(TYPE == 17 ? 66 : 74) + (sb >> 1)] >> (4 * (sb & 1))) & 15u;
  }

  static __device__ __forceinline__ uint8_t tile_byte(const FragSrc &s, long long p, int u, int b) {
    if (b < 1024) {
      const int pc = b >> 9, lane = (b & 511) >> 4, i = b & 15;
      const int g = lane >> 2, t = lane & 3, slot = i >> 2, bi = i & 3;
      const long long row = p * kFragRows + g + 8 * (slot & 1);
      if (row >= s.N) return 0;
      const int j = 2 * pc + (slot >> 1), sb = 4 * j + t;
      const uint8_t *blk = block(s, row, u);
      if (kWide) return blk[(bi < 2 ? 2 : 34) + 2 * sb + (bi & 1)];  // index bytes of the two entries, then their sign bytes
      return (uint8_t)(entry16(blk, 2 * sb + (bi >> 1)) >> (8 * (bi & 1)));
    }
    if (b < kD) {
      if (kWide) {
        const int idx = b - kScales, lane = idx >> 3, i = idx & 7;
        const int g = lane >> 2, t = lane & 3;
        const long long row = p * kFragRows + g + 8 * (i >> 2);
        if (row >= s.N) return 0;
        const uint8_t *blk = block(s, row, u);
        const int sb = 4 * (i & 3) + t;
        const uint32_t high = ((uint32_t)blk[66 + (sb >> 1)] >> (4 * (sb & 1))) & 15u;  // two bits per entry
        return (uint8_t)(scale4(blk, sb) | (high << 4));
      }
      const int idx = b - kScales, lane = idx >> 2, i = idx & 3;
      const int g = lane >> 2, t = lane & 3;
      const long long row = p * kFragRows + g + 8 * (i >> 1);
      if (row >= s.N) return 0;
      const uint8_t *blk = block(s, row, u);
      uint32_t out = 0;
      for (int e = 0; e < 2; ++e) {
        const int sb = 4 * (2 * (i & 1) + e) + t;  // nibble j = 2 (i & 1) + e of the lane's sixteen bits
        out |= scale4(blk, sb) << (4 * e);
      }
      return (uint8_t)out;
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

  // What does not depend on the launches before this one, set up ahead of the dependency wait:
  // the grid. Entry i = eight fp16 magnitudes (the codes are 2 bits each: 0, 1, 2 -> 8, 25, 43);
  // eight consecutive threads store the eight copies of an entry, 128 contiguous bytes.
  static __device__ __forceinline__ void before_wait(const FragArgs &a, uint32_t xfrag) {
    const uint32_t grid = xfrag + (uint32_t)a.umax * kXBytes + kGrid;
    for (int i = threadIdx.x; i < kEntries * kCopies; i += blockDim.x) {
      const int entry = i / kCopies;
      uint32_t w[4];
      if (TYPE == 17) {
        const uint32_t codes = g_iq2xs_frag_codes[entry];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const uint32_t c0 = (codes >> (4 * r)) & 3u, c1 = (codes >> (4 * r + 2)) & 3u;
          const uint32_t h0 = c0 == 0 ? 0x4800u : c0 == 1 ? 0x4e40u : 0x5160u;  // fp16 bits of 8, 25, 43
          const uint32_t h1 = c1 == 0 ? 0x4800u : c1 == 1 ? 0x4e40u : 0x5160u;
          w[r] = h0 | (h1 << 16);
        }
      } else {
        const uint64_t bytes = TYPE == 16 ? d_iq2xxs_grid[entry] : d_iq2s_grid[entry];  // eight magnitudes, a byte each
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const __half2 h = __halves2half2(__int2half_rn((int)((bytes >> (16 * r)) & 0xffull)),
                                           __int2half_rn((int)((bytes >> (16 * r + 8)) & 0xffull)));
          w[r] = *reinterpret_cast<const uint32_t *>(&h);
        }
      }
      sts128u(grid + (uint32_t)i * 16u, make_uint4(w[0], w[1], w[2], w[3]));
    }
  }

  // Activations of the CTA's column range as they lie in x (rows past M as zeros).
  // A warp task is (unit, activation row): lane l loads and stores k = 8l .. 8l + 7.
  // after_loads() runs once, when the first batch of loads is in flight. IQ2_XS has no rotation.
  template <class F>
  static __device__ __forceinline__ void stage_x(const FragArgs &a, uint32_t xfrag, int ub0, int uc, F &&after_loads) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const uint32_t R = row_stride(a);
    const int tasks = uc * 8;
    constexpr int kBatch = 8;
    const __half *xl = a.x + (long long)ub0 * 256 + lane * 8;
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
        sts128u(xfrag + (uint32_t)(i & 7) * R + (uint32_t)(i >> 3) * 512u + (uint32_t)lane * 16u, v[e]);
      }
    }
  }

  // 2 s + 1 of scale nibble j of the sixteen bits `nibbles`, in both halves of a half2
  static __device__ __forceinline__ __half2 scale_of(uint32_t nibbles, int j) {
    const uint32_t bits = ((nibbles >> (4 * j)) & 15u) * 0x00020002u + 0x64016401u;  // the bits of 1024 + 2 s + 1, twice
    return __hsub2(*reinterpret_cast<const __half2 *>(&bits), __float2half2_rn(1024.f));
  }

  // eight weights as four A registers, magnitude * (2 s + 1) * sign: index into the grid (this
  // lane's copy), the eight sign bits
  static __device__ __forceinline__ void entry(uint32_t (&r)[4], uint32_t index, uint32_t s8, uint32_t grid, __half2 scale) {
    const uint4 m = lds128(grid + index * (uint32_t)(kCopies * 16));
    const uint32_t mag[4] = {m.x, m.y, m.z, m.w};
    // sign bits 2r and 2r + 1 to bits 15 and 31
    const uint32_t mul[4] = {0x40008000u, 0x10002000u, 0x04000800u, 0x01000200u};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 v = __hmul2(*reinterpret_cast<const __half2 *>(&mag[i]), scale);
      r[i] = *reinterpret_cast<const uint32_t *>(&v) ^ ((s8 * mul[i]) & 0x80008000u);
    }
  }
  // the IQ2_XS form: nine index bits, seven sign bits and their parity as the eighth
  static __device__ __forceinline__ void entry(uint32_t (&r)[4], uint32_t q, uint32_t grid, __half2 scale) {
    const uint32_t s7 = (q >> 9) & 127u;
    entry(r, q & 511u, s7 | ((uint32_t)(__popc(s7) & 1) << 7), grid, scale);
  }

  // One tile against the activations of its unit; acc is the warp's C fragment.
  template <int MODE>
  static __device__ __forceinline__ void unit(float (&acc)[4], const FragArgs &a, uint32_t tile, uint32_t xbase, int uq,
                                              int g, int t, int lane) {
    const uint32_t R = row_stride(a);
    const uint32_t grid = xbase + (uint32_t)a.umax * kXBytes + kGrid + (uint32_t)(lane & (kCopies - 1)) * 16u;
    const uint32_t xrow = xbase + (uint32_t)g * R + (uint32_t)uq * 512u + (uint32_t)t * 32u;
    // scales: nibbles j of row g in the low half, of row g + 8 in the high half; IQ2_S: a byte per
    // sub-block (scale | high index bits << 4), row g in sw.x, row g + 8 in sw.y
    uint32_t sn = 0;
    uint2 sw = make_uint2(0u, 0u);
    if (kWide) sw = lds64(tile + kScales + (uint32_t)lane * 8u);
    else sn = lds32(tile + kScales + (uint32_t)lane * 4u);
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int pc = 0; pc < 2; ++pc) {
      const uint4 w = lds128(tile + (uint32_t)pc * 512u + (uint32_t)lane * 16u);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = 2 * pc + e;
        const uint32_t q0 = e ? w.z : w.x, q1 = e ? w.w : w.y;  // the sub-block's two entries of row g, of row g + 8
        uint32_t lo0[4], hi0[4], lo1[4], hi1[4];
        if (kWide) {
          const uint32_t b0 = sw.x >> (8 * j), b1 = sw.y >> (8 * j);
          const __half2 s0 = scale_of(b0, 0), s1 = scale_of(b1, 0);
          entry(lo0, (q0 & 0xffu) | ((b0 << 4) & 0x300u), (q0 >> 16) & 0xffu, grid, s0);
          entry(hi0, ((q0 >> 8) & 0xffu) | ((b0 << 2) & 0x300u), q0 >> 24, grid, s0);
          entry(lo1, (q1 & 0xffu) | ((b1 << 4) & 0x300u), (q1 >> 16) & 0xffu, grid, s1);
          entry(hi1, ((q1 >> 8) & 0xffu) | ((b1 << 2) & 0x300u), q1 >> 24, grid, s1);
        } else {
          const __half2 s0 = scale_of(sn, j), s1 = scale_of(sn >> 16, j);
          entry(lo0, q0 & 0xffffu, grid, s0);
          entry(hi0, q0 >> 16, grid, s0);
          entry(lo1, q1 & 0xffffu, grid, s1);
          entry(hi1, q1 >> 16, grid, s1);
        }
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
    const float d0 = half_bits_to_float(dd & 0xffffu) * 0.125f, d1 = half_bits_to_float(dd >> 16) * 0.125f;
    acc[0] = fmaf(d0, c[0], acc[0]);
    acc[1] = fmaf(d0, c[1], acc[1]);
    acc[2] = fmaf(d1, c[2], acc[2]);
    acc[3] = fmaf(d1, c[3], acc[3]);
  }
};

using FragIQ2XS = FragIQ2<17>;

}  // namespace ishi
