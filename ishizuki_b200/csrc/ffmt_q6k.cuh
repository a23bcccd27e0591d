// GGUF Q6_K for the warp-level kernel (mma.sync fragments).
//
// Block layout (210 bytes per 256 weights; reference: Sources/IshizukiKit/Core/GGMLDequant.swift,
// the Q6_K decoder, and the matvec body in Sources/IshizukiKit/Core/GGMLKernels.swift):
//   ql[128] low nibbles @0, qh[64] high bit pairs @128, sixteen int8 scales @192, d f16 @208.
//   Weight k = 128n + 32c + l (half n, quarter c, l < 32) has its low nibble in ql[64n + 32(c&1) + l]
//   (the high nibble of that byte when c >= 2) and its two high bits at bit 2c of qh[32n + l];
//   w = d * scale[k / 16] * (q - 32).
//
// The product is factored as
//   y += d * (sum_g scale_g * sum_{k in g} q_k x_k  -  32 * sum_g scale_g * sum_{k in g} x_k),
// g running over the sixteen groups of 16 weights. A group is exactly one k-step of the MMA, so
// every k-step's accumulator takes its (exact, fp32) scale afterwards; the second sum is one more
// MMA whose k index runs over the groups, against the group sums of x.
//
// A 6-bit value masked in place at bits 0..5 of each half of a register is the bit pattern of the
// fp16 number q * 2^-24; at bits 4..9 it is q * 2^-20 (both subnormal, hence linear in q). The tile
// stores the nibbles and the bit pairs where those masks find them:
//   a pair of k-steps (2i, 2i + 1) takes, per lane, one nibble word per weight row (X1: row g,
//   X2: row g + 8) and one word H of sixteen bit pairs. With Y = X >> 8, the k-step 2i uses
//   (X1, X2, Y1, Y2) & 0x000f000f as its four A registers and the k-step 2i + 1 uses the same words
//   & 0x00f000f0 (sixteen times too large; its scale is divided by 16). The high bits come from H
//   rotated right by 0, 2, 8 and 10: each rotation lines one pair of fields up with mask
//   0x00300030 (first k-step) and another with 0x03000300 (second k-step), so a register costs two
//   bit operations: (X & m) | (rot(H) & c).
// Inside a k-step the lane t holds the weights 4t .. 4t + 3 of the group: slots (2t, 2t + 1) are
// 4t, 4t + 1 and slots (2t + 8, 2t + 9) are 4t + 2, 4t + 3; the activations are staged in the same
// order, so that a lane reads the B registers of two k-steps with one 16-byte load.
//
// Tile (16 rows x 256 k, 3360 bytes = 16 * 210): nibble words [4][lane][X1 X2 | X1' X2'] @0,
// bit-pair words [4][lane][H H'] @2048, per row the sixteen scales @3072 in the order
// (2t, 2t + 1, 2t + 8, 2t + 9) for t = 0..3 (a lane's A registers of the group-sum MMA are then one
// word), and d of rows (g, g + 8) side by side @3328.
#pragma once
#include "ishi_fragstream.cuh"

namespace ishi {

struct FragQ6K {
  static constexpr int kTileBytes = 16 * 210;
  static constexpr int kXSums = 4096;             // after the activations: [lane][hi hi | lo lo] group sums
  static constexpr int kXBytes = kXSums + 512;    // per unit
  static constexpr int kExtraBytes = 0;  // shared memory per CTA beyond the per-unit staging
  static constexpr bool kRowMode = false;         // one activation row runs through the MMA path as well

  // the 6-bit code of weight k of a block
  static __device__ __forceinline__ uint32_t code(const uint8_t *blk, int k) {
    const int n = k >> 7, c = (k >> 5) & 3, l = k & 31;
    const uint32_t lo = blk[64 * n + 32 * (c & 1) + l];
    const uint32_t hi = blk[128 + 32 * n + l];
    return ((c >= 2 ? lo >> 4 : lo) & 15u) | (((hi >> (2 * c)) & 3u) << 4);
  }

  static __device__ __forceinline__ const uint8_t *block(const FragSrc &s, long long row, int u) {
    long long local;
    const int seg = frag_segment(s, row, &local);
    return s.w[seg] + local * s.w_row_bytes + (long long)u * 210;
  }

  static __device__ __forceinline__ uint8_t tile_byte(const FragSrc &s, long long p, int u, int b) {
    if (b < 2048) {
      const int pp = b >> 9, lane = (b & 511) >> 4, i = b & 15;
      const int g = lane >> 2, t = lane & 3, w = i >> 2, bi = i & 3;
      const long long row = p * kFragRows + g + 8 * (w & 1);
      if (row >= s.N) return 0;
      const uint8_t *blk = block(s, row, u);
      const int pi = 2 * pp + (w >> 1);
      uint32_t out = 0;
      for (int e = 0; e < 2; ++e) {
        const int n = 2 * bi + e;  // nibble of the word
        const int ks = 2 * pi + (n & 1), kk = 4 * t + 2 * ((n >> 1) & 1) + (n >> 2);
        out |= (code(blk, 16 * ks + kk) & 15u) << (4 * e);
      }
      return (uint8_t)out;
    }
    if (b < 3072) {
      const int idx = b - 2048, pp = idx >> 8, lane = (idx & 255) >> 3, i = idx & 7;
      const int g = lane >> 2, t = lane & 3, pi = 2 * pp + (i >> 2), bi = i & 3;
      uint32_t out = 0;
      for (int e = 0; e < 4; ++e) {
        const int pos = 8 * bi + 2 * e;  // bit position of the field in H
        // which register's half the field feeds: rotation r lines positions 4 + r, 20 + r (first
        // k-step) and 8 + r, 24 + r (second) up with the masks; r = 0, 2 serve row g (X, Y), 8, 10 row g + 8
        int second, y, x2, half;
        const int q = pos & 15;  // position modulo the halves
        if (q == 4 || q == 6) second = 0, x2 = 0, y = q == 6, half = pos >> 4;
        else if (q == 8 || q == 10) second = 1, x2 = 0, y = q == 10, half = pos >> 4;
        else if (q == 12 || q == 14) second = 0, x2 = 1, y = q == 14, half = pos >> 4;
        else second = 1, x2 = 1, y = q == 2, half = 1 - (pos >> 4);  // positions 16, 18 | 0, 2: rotated across the halves
        const long long row = p * kFragRows + g + 8 * x2;
        if (row >= s.N) continue;
        const int ks = 2 * pi + second, kk = 4 * t + 2 * y + half;
        out |= (code(block(s, row, u), 16 * ks + kk) >> 4) << (2 * e);
      }
      return (uint8_t)out;
    }
    if (b < 3328) {
      const int idx = b - 3072, j = idx & 15;
      const long long row = p * kFragRows + (idx >> 4);
      if (row >= s.N) return 0;
      const int ks = 2 * (j >> 2) + (j & 1) + 8 * ((j >> 1) & 1);
      return block(s, row, u)[192 + ks];
    }
    const int idx = b - 3328;
    const long long row = p * kFragRows + (idx >> 2) + 8 * ((idx >> 1) & 1);
    if (row >= s.N) return 0;
    return block(s, row, u)[208 + (idx & 1)];
  }

  static __device__ __forceinline__ uint16_t tile_halfword(const FragSrc &s, long long p, int u, int hw) {
    return (uint16_t)(tile_byte(s, p, u, 2 * hw) | ((uint32_t)tile_byte(s, p, u, 2 * hw + 1) << 8));
  }

  // nothing to set up ahead of the dependency wait
  static __device__ __forceinline__ void before_wait(const FragArgs &, uint32_t) {}

  // Activations of the CTA's column range into fragment order. A warp task is (unit, activation
  // row r): lane l loads k = 8l .. 8l + 7, half of group l / 2, i.e. what lanes t = 2(l & 1) and
  // t + 1 of quad r multiply in k-step l / 2. The pair of k-steps i = l / 4 lies at
  // i * 512 + ((r ^ i) * 4 + t) * 16 (+ 8 for the odd k-step); the xor spreads the stores over the
  // banks and a warp's read of one pair is still one 512-byte run. Then the group sums (fp16 hi +
  // lo) for the MMA over groups. after_loads() runs once, when the first loads are in flight.
  template <class F>
  static __device__ __forceinline__ void stage_x(const FragArgs &a, uint32_t xfrag, int ub0, int uc, F &&after_loads) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
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
        const int r = i & 7, u = i >> 3;
        const uint32_t base = xfrag + (uint32_t)u * kXBytes;
        const int pi = lane >> 2, ks = lane >> 1;
        const uint32_t dst = base + (uint32_t)pi * 512u + (uint32_t)(((r ^ pi) * 4 + 2 * (lane & 1)) * 16 + (ks & 1) * 8);
        sts64(dst, v[e].x, v[e].y);
        sts64(dst + 16u, v[e].z, v[e].w);
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].y));
        const float2 f2 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].z));
        const float2 f3 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].w));
        float s = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
        s += __shfl_xor_sync(0xffffffffu, s, 1);  // the group's sixteen values
        if ((lane & 1) == 0) {
          const __half hi = __float2half_rn(s), lo = __float2half_rn(s - __half2float(hi));
          // group ks is slot ks of the MMA over groups: lane t' = (ks % 8) / 2 of quad r holds it in
          // register ks / 8, half ks % 2
          const uint32_t at = base + kXSums + (uint32_t)((r * 4 + ((ks & 7) >> 1)) * 16 + (ks >> 3) * 4 + (ks & 1) * 2);
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(at), "h"(__half_as_ushort(hi)) : "memory");
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(at + 8u), "h"(__half_as_ushort(lo)) : "memory");
        }
      }
    }
  }

  static __device__ __forceinline__ float scale_of(uint32_t word, int byte) {
    return (float)(int)(int8_t)(word >> (8 * byte));
  }
  // two int8 of a word (already xor 0x80 per byte) as a half2: the bits of 1024 + 128 + b, minus 1152
  static __device__ __forceinline__ uint32_t scale_pair(uint32_t biased, uint32_t selector) {
    const uint32_t bits = prmt(biased, 0x64646464u, selector);
    const __half2 v = __hsub2(*reinterpret_cast<const __half2 *>(&bits), __float2half2_rn(1152.f));
    return *reinterpret_cast<const uint32_t *>(&v);
  }

  // One tile against the activations of its unit; acc is the warp's C fragment.
  template <int MODE>
  static __device__ __forceinline__ void unit(float (&acc)[4], const FragArgs &a, uint32_t tile, uint32_t xbase, int uq,
                                              int g, int t, int lane) {
    (void)a;
    const uint32_t xu = xbase + (uint32_t)uq * kXBytes;
    const uint4 h0 = lds128(tile + 3072u + (uint32_t)g * 16u), h1 = lds128(tile + 3072u + (uint32_t)(g + 8) * 16u);
    const uint32_t hw0[4] = {h0.x, h0.y, h0.z, h0.w}, hw1[4] = {h1.x, h1.y, h1.z, h1.w};
    const uint32_t lane_off = (uint32_t)g * 64u + (uint32_t)t * 16u;
    float su[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int pp = 0; pp < 4; ++pp) {
      const uint4 q = lds128(tile + (uint32_t)pp * 512u + (uint32_t)lane * 16u);
      const uint2 hh = lds64(tile + 2048u + (uint32_t)pp * 256u + (uint32_t)lane * 8u);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int pi = 2 * pp + e;
        const uint32_t x1 = e ? q.z : q.x, x2 = e ? q.w : q.y, h = e ? hh.y : hh.x;
        const uint4 b = lds128(xu + (uint32_t)pi * 512u + (lane_off ^ (uint32_t)(pi << 6)));
        const uint32_t y1 = x1 >> 8, y2 = x2 >> 8;
        const uint32_t r2 = __funnelshift_r(h, h, 2), r8 = __funnelshift_r(h, h, 8), r10 = __funnelshift_r(h, h, 10);
        float c0[4], c1[4];
        mma16816_first(c0, (x1 & 0x000f000fu) | (h & 0x00300030u), (x2 & 0x000f000fu) | (r8 & 0x00300030u),
                       (y1 & 0x000f000fu) | (r2 & 0x00300030u), (y2 & 0x000f000fu) | (r10 & 0x00300030u), b.x, b.y);
        mma16816_first(c1, (x1 & 0x00f000f0u) | (h & 0x03000300u), (x2 & 0x00f000f0u) | (r8 & 0x03000300u),
                       (y1 & 0x00f000f0u) | (r2 & 0x03000300u), (y2 & 0x00f000f0u) | (r10 & 0x03000300u), b.z, b.w);
        // scales of groups 2 pi and 2 pi + 1: word pi % 4 of the row's sixteen, bytes 2 (pi / 4) and + 1
        const float s00 = scale_of(hw0[pi & 3], 2 * (pi >> 2)), s01 = scale_of(hw0[pi & 3], 2 * (pi >> 2) + 1) * 0.0625f;
        const float s10 = scale_of(hw1[pi & 3], 2 * (pi >> 2)), s11 = scale_of(hw1[pi & 3], 2 * (pi >> 2) + 1) * 0.0625f;
        su[0] = fmaf(s00, c0[0], su[0]), su[1] = fmaf(s00, c0[1], su[1]);
        su[2] = fmaf(s10, c0[2], su[2]), su[3] = fmaf(s10, c0[3], su[3]);
        su[0] = fmaf(s01, c1[0], su[0]), su[1] = fmaf(s01, c1[1], su[1]);
        su[2] = fmaf(s11, c1[2], su[2]), su[3] = fmaf(s11, c1[3], su[3]);
      }
    }
    // sum_g scale_g * (sum of x over group g): the MMA over groups; this lane's slots are groups
    // 2t, 2t + 1, 2t + 8, 2t + 9, the word t of each row's scales
    const uint32_t w0 = (t == 0 ? h0.x : t == 1 ? h0.y : t == 2 ? h0.z : h0.w) ^ 0x80808080u;
    const uint32_t w1 = (t == 0 ? h1.x : t == 1 ? h1.y : t == 2 ? h1.z : h1.w) ^ 0x80808080u;
    const uint4 bs = lds128(xu + kXSums + (uint32_t)lane * 16u);
    float cm[4];
    const uint32_t a0 = scale_pair(w0, 0x4140u), a1 = scale_pair(w1, 0x4140u);
    const uint32_t a2 = scale_pair(w0, 0x4342u), a3 = scale_pair(w1, 0x4342u);
    mma16816_first(cm, a0, a1, a2, a3, bs.x, bs.y);
    mma16816(cm, a0, a1, a2, a3, bs.z, bs.w);
    const uint32_t dd = lds32(tile + 3328u + (uint32_t)g * 4u);
    const float d0 = half_bits_to_float(dd & 0xffffu), d1 = half_bits_to_float(dd >> 16);
    const float dl0 = d0 * 16777216.f, dl1 = d1 * 16777216.f, dm0 = d0 * -32.f, dm1 = d1 * -32.f;
    acc[0] = fmaf(dl0, su[0], fmaf(dm0, cm[0], acc[0]));
    acc[1] = fmaf(dl0, su[1], fmaf(dm0, cm[1], acc[1]));
    acc[2] = fmaf(dl1, su[2], fmaf(dm1, cm[2], acc[2]));
    acc[3] = fmaf(dl1, su[3], fmaf(dm1, cm[3], acc[3]));
  }
};

}  // namespace ishi
