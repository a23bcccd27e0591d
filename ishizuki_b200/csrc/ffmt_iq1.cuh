// GGUF IQ1_S and IQ1_M for the warp-level kernel (mma.sync fragments).
//
// Block layouts (reference: Sources/IshizukiKit/Core/GGMLDequant.swift:376-428). Eight weights are
// one entry of a 2048-entry grid of values out of {-1, 0, 1}, plus a common delta of +-1/8:
//   w = d * (2 s + 1) * (grid value + delta).
//   IQ1_S (50 bytes per 256 weights): d f16 @0, 32 index bytes @2, eight words @34 per 32 weights:
//     three more index bits for each of the four entries, the scale s (3 bits), the delta's sign.
//   IQ1_M (56 bytes): 32 index bytes @0, 16 bytes @32 (per entry a nibble: three index bits and the
//     delta's sign), four words @48: 3-bit scales per sixteen weights, and in their top nibbles the
//     fp16 d.
//
// The product is factored as
//   y += d * (sum_k (2 s + 1) g_k x_k  +  1/8 * sum_E (+-(2 s + 1))_E * sum_{k in E} x_k),
// E running over the 32 entries of a unit. The first sum is the IQ2_XS scheme: the grid lives in
// shared memory (an entry = eight bytes value + 128, four copies, copy c of entry i at
// i * 32 + c * 8), two bytes become an fp16 pair by a byte permute (the bits of 1152 + v) and one
// fused multiply-add, (1152 + v) * (2 s + 1) - 1152 * (2 s + 1), exact. The second sum is two more
// k-steps of MMA over the entries, against the entries' sums of x (fp16 high and low parts): a
// lane's eight entries per row are exactly its A registers of those two k-steps.
//
// Fragment mapping as for IQ2_XS: a lane owns the sub-blocks (sixteen weights = two entries)
// 4 j + t, j = 0..3, of rows g and g + 8. Both formats are tiled into one form, a word per sub-block
// and row: index bytes of its two entries, their three high index bits (bits 16-18, 19-21), the
// scale (bits 24-26), the entries' delta signs (bits 27, 28). Tile (16 rows x 256 k, 1056 bytes;
// the blocks are 800 and 896): [2][lane][16 bytes] = for j = 2p, 2p + 1: the word of row g, of
// row g + 8; then d of rows (g, g + 8) side by side.
//
// Activations of a unit in shared memory: eight rows of 256 fp16 as they lie in x, the rows
// umax * 512 + 16 bytes apart; behind all rows, per unit, the entry sums: [k-step][lane][hi hi | lo lo].
#pragma once
#include "ggml_decode.cuh"
#include "ishi_fragstream.cuh"

namespace ishi {

// TYPE: the GGML type number, 19 IQ1_S, 29 IQ1_M
template <int TYPE>
struct FragIQ1 {
  static_assert(TYPE == 19 || TYPE == 29, "IQ1_S or IQ1_M");
  static constexpr int kBlock = TYPE == 19 ? 50 : 56;
  static constexpr int kD = 1024;
  static constexpr int kTileBytes = kD + 32;
  static constexpr int kXBytes = 8 * 512 + 1024;  // per unit: eight rows of 512 bytes, and the entry sums
  static constexpr int kGrid = 8 * 16;            // first in the extra region: the rows' 16-byte skews
  static constexpr int kExtraBytes = kGrid + 2048 * 32;  // then the grid, four copies interleaved
  static constexpr bool kRowMode = false;         // one activation row runs through the MMA path as well

  static __device__ __forceinline__ const uint8_t *block(const FragSrc &s, long long row, int u) {
    long long local;
    const int seg = frag_segment(s, row, &local);
    return s.w[seg] + local * s.w_row_bytes + (long long)u * kBlock;
  }
  static __device__ __forceinline__ uint32_t u16_at(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8); }

  // byte `bi` of the word of sub-block sb of a block (see above)
  static __device__ __forceinline__ uint8_t word_byte(const uint8_t *blk, int sb, int bi) {
    const int ib = sb >> 1, l0 = 2 * (sb & 1);  // the 32-group, the first of the sub-block's two entries in it
    if (TYPE == 19) {
      const uint32_t qh = u16_at(blk + 34 + 2 * ib);
      if (bi < 2) return blk[2 + 4 * ib + l0 + bi];
      if (bi == 2) return (uint8_t)((qh >> (3 * l0)) & 63u);
      return (uint8_t)(((qh >> 12) & 7u) | ((qh >> 15) << 3) | ((qh >> 15) << 4));
    }
    const uint32_t qhb = blk[32 + 2 * ib + (l0 >> 1)];  // low nibble: the first entry, high nibble: the second
    if (bi < 2) return blk[4 * ib + l0 + bi];
    if (bi == 2) return (uint8_t)((qhb & 7u) | (((qhb >> 4) & 7u) << 3));
    const uint32_t scale = (u16_at(blk + 48 + 2 * (ib >> 1)) >> (6 * (ib & 1) + 3 * (sb & 1))) & 7u;
    return (uint8_t)(scale | (((qhb >> 3) & 1u) << 3) | (((qhb >> 7) & 1u) << 4));
  }

  static __device__ __forceinline__ uint8_t tile_byte(const FragSrc &s, long long p, int u, int b) {
    if (b < kD) {
      const int pc = b >> 9, lane = (b & 511) >> 4, i = b & 15;
      const int g = lane >> 2, t = lane & 3, slot = i >> 2, bi = i & 3;
      const long long row = p * kFragRows + g + 8 * (slot & 1);
      if (row >= s.N) return 0;
      return word_byte(block(s, row, u), 4 * (2 * pc + (slot >> 1)) + t, bi);
    }
    const int idx = b - kD;
    const long long row = p * kFragRows + (idx >> 2) + 8 * ((idx >> 1) & 1);
    if (row >= s.N) return 0;
    const uint8_t *blk = block(s, row, u);
    if (TYPE == 19) return blk[idx & 1];
    const uint32_t s0 = u16_at(blk + 48), s1 = u16_at(blk + 50), s2 = u16_at(blk + 52), s3 = u16_at(blk + 54);
    const uint32_t d = (s0 >> 12) | ((s1 >> 8) & 0x00f0u) | ((s2 >> 4) & 0x0f00u) | (s3 & 0xf000u);
    return (uint8_t)(d >> (8 * (idx & 1)));
  }

  static __device__ __forceinline__ uint16_t tile_halfword(const FragSrc &s, long long p, int u, int hw) {
    return (uint16_t)(tile_byte(s, p, u, 2 * hw) | ((uint32_t)tile_byte(s, p, u, 2 * hw + 1) << 8));
  }

  static __device__ __forceinline__ uint32_t row_stride(const FragArgs &a) { return (uint32_t)a.umax * 512u + 16u; }
  // the entry sums of unit u: behind the eight rows
  static __device__ __forceinline__ uint32_t sums_of(const FragArgs &a, uint32_t xfrag, int u) {
    return xfrag + (uint32_t)a.umax * 4096u + 128u + (uint32_t)u * 1024u;
  }

  // the grid (each value + 128), set up ahead of the dependency wait; four consecutive threads
  // store the four copies of an entry
  static __device__ __forceinline__ void before_wait(const FragArgs &a, uint32_t xfrag) {
    const uint32_t grid = xfrag + (uint32_t)a.umax * kXBytes + kGrid;
    for (int i = threadIdx.x; i < 2048 * 4; i += blockDim.x) {
      const uint64_t v = d_iq1s_grid[i >> 2] ^ 0x8080808080808080ull;
      sts64(grid + (uint32_t)i * 8u, (uint32_t)v, (uint32_t)(v >> 32));
    }
  }

  // Activations of the CTA's column range as they lie in x (rows past M as zeros), and per entry
  // (the eight values of one lane) their sum as fp16 high and low parts, where the MMA over the
  // entries reads them: entry E = 2 (4 j + t) + e is slot 2t + e + 8 (j % 2) of k-step j / 2, i.e.
  // register j % 2, half e, of lane (r, t). after_loads() runs once, when the first batch of loads
  // is in flight. No rotation here.
  template <class F>
  static __device__ __forceinline__ void stage_x(const FragArgs &a, uint32_t xfrag, int ub0, int uc, F &&after_loads) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const uint32_t R = row_stride(a);
    const int tasks = uc * 8;
    constexpr int kBatch = 8;
    const __half *xl = a.x + (long long)ub0 * 256 + lane * 8;
    const int sb = lane >> 1, j = sb >> 2, t = sb & 3;
    const uint32_t slot = (uint32_t)((j >> 1) * 512 + t * 16 + (j & 1) * 4 + (lane & 1) * 2);
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
        const int r = i & 7, u = i >> 3;
        sts128u(xfrag + (uint32_t)r * R + (uint32_t)u * 512u + (uint32_t)lane * 16u, v[e]);
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].y));
        const float2 f2 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].z));
        const float2 f3 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].w));
        const float s = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
        const __half hi = __float2half_rn(s), lo = __float2half_rn(s - __half2float(hi));
        const uint32_t at = sums_of(a, xfrag, u) + (uint32_t)r * 64u + slot;
        asm volatile("st.shared.u16 [%0], %1;" ::"r"(at), "h"(__half_as_ushort(hi)) : "memory");
        asm volatile("st.shared.u16 [%0], %1;" ::"r"(at + 8u), "h"(__half_as_ushort(lo)) : "memory");
      }
    }
  }

  // eight weights as four A registers, value * (2 s + 1): the grid index (this lane's copy of the
  // grid), scale = 2 s + 1 and offset = -1152 * (2 s + 1) in both halves
  static __device__ __forceinline__ void entry(uint32_t (&r)[4], uint32_t index, uint32_t grid, __half2 scale, __half2 offset) {
    const uint2 m = lds64(grid + index * 32u);
    const uint32_t bits[4] = {prmt(m.x, 0x64646464u, 0x4140u), prmt(m.x, 0x64646464u, 0x4342u), prmt(m.y, 0x64646464u, 0x4140u),
                              prmt(m.y, 0x64646464u, 0x4342u)};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 v = __hfma2(*reinterpret_cast<const __half2 *>(&bits[i]), scale, offset);
      r[i] = *reinterpret_cast<const uint32_t *>(&v);
    }
  }

  // One tile against the activations of its unit; acc is the warp's C fragment.
  template <int MODE>
  static __device__ __forceinline__ void unit(float (&acc)[4], const FragArgs &a, uint32_t tile, uint32_t xbase, int uq,
                                              int g, int t, int lane) {
    const uint32_t R = row_stride(a);
    const uint32_t grid = xbase + (uint32_t)a.umax * kXBytes + kGrid + (uint32_t)(lane & 3) * 8u;
    const uint32_t xrow = xbase + (uint32_t)g * R + (uint32_t)uq * 512u + (uint32_t)t * 32u;
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    uint32_t da[2][4];  // the A registers of the two k-steps over the entries: +-(2 s + 1)
#pragma unroll
    for (int pc = 0; pc < 2; ++pc) {
      const uint4 w = lds128(tile + (uint32_t)pc * 512u + (uint32_t)lane * 16u);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = 2 * pc + e;
        const uint32_t q0 = e ? w.z : w.x, q1 = e ? w.w : w.y;  // the sub-block's word of row g, of row g + 8
        uint32_t lo0[4], hi0[4], lo1[4], hi1[4];
        const uint32_t b0 = ((q0 >> 24) & 7u) * 0x00020002u + 0x64016401u, b1 = ((q1 >> 24) & 7u) * 0x00020002u + 0x64016401u;
        const __half2 s0 = __hsub2(*reinterpret_cast<const __half2 *>(&b0), __float2half2_rn(1024.f));
        const __half2 s1 = __hsub2(*reinterpret_cast<const __half2 *>(&b1), __float2half2_rn(1024.f));
        const __half2 o0 = __hmul2(s0, __float2half2_rn(-1152.f)), o1 = __hmul2(s1, __float2half2_rn(-1152.f));
        entry(lo0, (q0 & 0xffu) | ((q0 >> 8) & 0x700u), grid, s0, o0);
        entry(hi0, ((q0 >> 8) & 0xffu) | ((q0 >> 11) & 0x700u), grid, s0, o0);
        entry(lo1, (q1 & 0xffu) | ((q1 >> 8) & 0x700u), grid, s1, o1);
        entry(hi1, ((q1 >> 8) & 0xffu) | ((q1 >> 11) & 0x700u), grid, s1, o1);
        // the two entries' +-(2 s + 1): the delta's sign bits 27 and 28 to bits 15 and 31
        da[j >> 1][(j & 1) * 2] = *reinterpret_cast<const uint32_t *>(&s0) ^ (((q0 >> 12) & 0x8000u) | ((q0 << 3) & 0x80000000u));
        da[j >> 1][(j & 1) * 2 + 1] = *reinterpret_cast<const uint32_t *>(&s1) ^ (((q1 >> 12) & 0x8000u) | ((q1 << 3) & 0x80000000u));
        const uint4 x0 = lds128(xrow + (uint32_t)j * 128u), x1 = lds128(xrow + (uint32_t)j * 128u + 16u);
        if (j == 0)
          mma16816_first(c, lo0[0], lo1[0], lo0[1], lo1[1], x0.x, x0.y);
        else
          mma16816(c, lo0[0], lo1[0], lo0[1], lo1[1], x0.x, x0.y);
        mma16816(c, lo0[2], lo1[2], lo0[3], lo1[3], x0.z, x0.w);
        mma16816(c, hi0[0], hi1[0], hi0[1], hi1[1], x1.x, x1.y);
        mma16816(c, hi0[2], hi1[2], hi0[3], hi1[3], x1.z, x1.w);
      }
    }
    // sum_E +-(2 s + 1) * (sum of x over entry E): da[ks] = {row g: j = 2 ks, row g + 8: j = 2 ks,
    // row g: j = 2 ks + 1, row g + 8: j = 2 ks + 1} = the registers a0, a1, a2, a3 of k-step ks
    const uint32_t sums = sums_of(a, xbase, uq) + (uint32_t)lane * 16u;
    float cm[4];
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      const uint4 bs = lds128(sums + (uint32_t)ks * 512u);
      if (ks == 0) mma16816_first(cm, da[ks][0], da[ks][1], da[ks][2], da[ks][3], bs.x, bs.y);
      else mma16816(cm, da[ks][0], da[ks][1], da[ks][2], da[ks][3], bs.x, bs.y);
      mma16816(cm, da[ks][0], da[ks][1], da[ks][2], da[ks][3], bs.z, bs.w);
    }
    const uint32_t dd = lds32(tile + (uint32_t)kD + (uint32_t)g * 4u);
    const float d0 = half_bits_to_float(dd & 0xffffu), d1 = half_bits_to_float(dd >> 16);
    acc[0] = fmaf(d0, fmaf(0.125f, cm[0], c[0]), acc[0]);
    acc[1] = fmaf(d0, fmaf(0.125f, cm[1], c[1]), acc[1]);
    acc[2] = fmaf(d1, fmaf(0.125f, cm[2], c[2]), acc[2]);
    acc[3] = fmaf(d1, fmaf(0.125f, cm[3], c[3]), acc[3]);
  }
};

}  // namespace ishi
