// GGUF Q2_K for the warp-level kernel (mma.sync fragments).
//
// Block layout (84 bytes per 256 weights; reference: Sources/IshizukiKit/Core/GGMLDequant.swift:125-150):
//   sixteen bytes (scale | min << 4) @0, 64 code bytes @16, d f16 @80, dmin f16 @82. Weight
//   k = 128 n + 32 j + l (half n, shift j < 4, l < 32) has its two bits at bit 2j of code byte
//   32 n + l and belongs to sub-block is = 8 n + 2 j + l / 16;  w = d * scale_is * q - dmin * min_is.
//
// The product is factored as
//   y += d * sum_is scale_is * sum_{k in is} q_k x_k  -  dmin * sum_is min_is * sum_{k in is} x_k.
// A sub-block is exactly one k-step of the MMA, so every k-step's accumulator takes its (integer)
// scale afterwards; the second sum is one more MMA whose k index runs over the sub-blocks, against
// the sub-block sums of x (fp16 high and low parts).
//
// A 2-bit code masked in place at bits 2j, 2j + 1 of each half of a register is the bit pattern of
// the fp16 number q * 4^j * 2^-24 (subnormal, hence linear in q); the activations of shift j are
// staged divided by 4^j (exact unless |x| is tiny). A lane t owns, per weight row, the 32-bit word
// of code bytes 32 n + 16 h + 4t .. + 3 (h = l / 16): masked at shift j it gives the weights
// l % 16 = 4t, 4t + 2 of sub-block 8 n + 2 j + h, shifted right by 8 and masked the weights 4t + 1,
// 4t + 3: the MMA's k columns (2t, 2t + 1) and (2t + 8, 2t + 9); the activations are staged in that order.
//
// Tile (16 rows x 256 k, 1344 bytes = 16 * 84): code words [2][lane][row g: h = 0, 1; row g + 8:
// h = 0, 1] @0, per row the sixteen scale bytes @1024 in the order (2t, 2t + 1, 2t + 8, 2t + 9) for
// t = 0..3 (a lane's A registers of the MMA over sub-blocks are then one word), d of rows
// (g, g + 8) side by side @1280, dmin the same @1312.
#pragma once
#include "ishi_fragstream.cuh"

namespace ishi {

struct FragQ2K {
  static constexpr int kTileBytes = 16 * 84;
  static constexpr int kXSums = 4096;           // after the activations: [lane][hi hi | lo lo] sub-block sums
  static constexpr int kXBytes = kXSums + 512;  // per unit
  static constexpr int kExtraBytes = 0;
  static constexpr bool kRowMode = false;       // one activation row runs through the MMA path as well

  static __device__ __forceinline__ const uint8_t *block(const FragSrc &s, long long row, int u) {
    long long local;
    const int seg = frag_segment(s, row, &local);
    return s.w[seg] + local * s.w_row_bytes + (long long)u * 84;
  }

  static __device__ __forceinline__ uint8_t tile_byte(const FragSrc &s, long long p, int u, int b) {
    if (b < 1024) {
      const int n = b >> 9, lane = (b & 511) >> 4, i = b & 15;
      const int g = lane >> 2, t = lane & 3, wi = i >> 2, bi = i & 3;
      const long long row = p * kFragRows + g + 8 * (wi >> 1);
      if (row >= s.N) return 0;
      return block(s, row, u)[16 + 32 * n + 16 * (wi & 1) + 4 * t + bi];
    }
    if (b < 1280) {
      const int idx = b - 1024, pos = idx & 15;
      const long long row = p * kFragRows + (idx >> 4);
      if (row >= s.N) return 0;
      const int is = 2 * (pos >> 2) + (pos & 1) + 8 * ((pos >> 1) & 1);
      return block(s, row, u)[is];
    }
    const int idx = (b - 1280) & 31;
    const long long row = p * kFragRows + (idx >> 2) + 8 * ((idx >> 1) & 1);
    if (row >= s.N) return 0;
    return block(s, row, u)[(b < 1312 ? 80 : 82) + (idx & 1)];
  }

  static __device__ __forceinline__ uint16_t tile_halfword(const FragSrc &s, long long p, int u, int hw) {
    return (uint16_t)(tile_byte(s, p, u, 2 * hw) | ((uint32_t)tile_byte(s, p, u, 2 * hw + 1) << 8));
  }

  // nothing to set up ahead of the dependency wait
  static __device__ __forceinline__ void before_wait(const FragArgs &, uint32_t) {}

  // Activations of the CTA's column range into fragment order. A warp task is (unit, activation
  // row r): lane l loads k = 8l .. 8l + 7: half n = l / 16, shift j = (l / 4) % 4, h = (l % 4) / 2,
  // the weights l % 16 = 8 (l % 2) ... + 7 of sub-block is = 8 n + 2 j + h, i.e. what lanes
  // t = 2 (l % 2) and t + 1 of quad r multiply in k-step is; stored divided by 4^j at
  // is * 256 + ((r ^ (is % 8)) * 4 + t) * 8 (the xor spreads the stores over the banks, a warp's read
  // of one k-step is still one 256-byte run). Then the sub-block sums of the undivided values
  // (fp16 hi + lo) for the MMA over sub-blocks. after_loads() runs once, when the first loads are
  // in flight. No rotation here.
  template <class F>
  static __device__ __forceinline__ void stage_x(const FragArgs &a, uint32_t xfrag, int ub0, int uc, F &&after_loads) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int tasks = uc * 8;
    constexpr int kBatch = 8;
    const __half *xl = a.x + (long long)ub0 * 256 + lane * 8;
    const int j = (lane >> 2) & 3;
    const int is = 8 * (lane >> 4) + 2 * j + ((lane & 3) >> 1);
    const uint32_t down1 = (uint32_t)(15 - 2 * j) << 10;  // 4^-j in fp16
    const uint32_t down = down1 | (down1 << 16);
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
        const __half2 dn = *reinterpret_cast<const __half2 *>(&down);
        // (x0 x2), (x1 x3) for t = 2 (l % 2); (x4 x6), (x5 x7) for t + 1
        uint32_t w[4] = {prmt(v[e].x, v[e].y, 0x5410u), prmt(v[e].x, v[e].y, 0x7632u), prmt(v[e].z, v[e].w, 0x5410u),
                         prmt(v[e].z, v[e].w, 0x7632u)};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const __half2 h = __hmul2(*reinterpret_cast<const __half2 *>(&w[q]), dn);
          w[q] = *reinterpret_cast<const uint32_t *>(&h);
        }
        sts128u(base + (uint32_t)is * 256u + (uint32_t)(((r ^ (is & 7)) * 4 + 2 * (lane & 1)) * 8), make_uint4(w[0], w[1], w[2], w[3]));
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].y));
        const float2 f2 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].z));
        const float2 f3 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].w));
        float s = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
        s += __shfl_xor_sync(0xffffffffu, s, 1);  // the sub-block's sixteen values
        if ((lane & 1) == 0) {
          const __half hi = __float2half_rn(s), lo = __float2half_rn(s - __half2float(hi));
          // sub-block is is slot is of the MMA over sub-blocks: lane t' = (is % 8) / 2 of quad r holds
          // it in register is / 8, half is % 2
          const uint32_t at = base + kXSums + (uint32_t)((r * 4 + ((is & 7) >> 1)) * 16 + (is >> 3) * 4 + (is & 1) * 2);
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(at), "h"(__half_as_ushort(hi)) : "memory");
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(at + 8u), "h"(__half_as_ushort(lo)) : "memory");
        }
      }
    }
  }

  // 8388608 + byte `byte` of word w, as a float
  static __device__ __forceinline__ float byte_float(uint32_t w, int byte) {
    return __uint_as_float(prmt(w, 0x4b000000u, 0x7440u | (uint32_t)byte));
  }
  // two bytes (each < 16) of a word as a half2: the bits of 1024 + b, minus 1024
  static __device__ __forceinline__ uint32_t byte_pair(uint32_t w, uint32_t selector) {
    const uint32_t bits = prmt(w, 0x64646464u, selector);
    const __half2 v = __hsub2(*reinterpret_cast<const __half2 *>(&bits), __float2half2_rn(1024.f));
    return *reinterpret_cast<const uint32_t *>(&v);
  }

  // One tile against the activations of its unit; acc is the warp's C fragment.
  template <int MODE>
  static __device__ __forceinline__ void unit(float (&acc)[4], const FragArgs &a, uint32_t tile, uint32_t xbase, int uq,
                                              int g, int t, int lane) {
    (void)a;
    const uint32_t xu = xbase + (uint32_t)uq * kXBytes;
    const uint4 h0 = lds128(tile + 1024u + (uint32_t)g * 16u), h1 = lds128(tile + 1024u + (uint32_t)(g + 8) * 16u);
    // the scales (low nibbles), word tw = sub-blocks (2 tw, 2 tw + 1, 2 tw + 8, 2 tw + 9)
    const uint32_t sl0[4] = {h0.x & 0x0f0f0f0fu, h0.y & 0x0f0f0f0fu, h0.z & 0x0f0f0f0fu, h0.w & 0x0f0f0f0fu};
    const uint32_t sl1[4] = {h1.x & 0x0f0f0f0fu, h1.y & 0x0f0f0f0fu, h1.z & 0x0f0f0f0fu, h1.w & 0x0f0f0f0fu};
    const uint32_t xl = xu + (uint32_t)t * 8u;
    float su[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const uint4 q = lds128(tile + (uint32_t)n * 512u + (uint32_t)lane * 16u);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t w0 = h ? q.y : q.x, w1 = h ? q.w : q.z;
        const uint32_t y0 = w0 >> 8, y1 = w1 >> 8;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int is = 8 * n + 2 * j + h;
          const uint32_t mask = 0x00030003u << (2 * j);
          const uint2 b = lds64(xl + (uint32_t)is * 256u + (uint32_t)((g ^ (is & 7)) * 32));
          float part[4];
          mma16816_first(part, w0 & mask, w1 & mask, y0 & mask, y1 & mask, b.x, b.y);
          const int tw = (is & 7) >> 1, e = (is & 1) + 2 * (is >> 3);
          const float f0 = byte_float(sl0[tw], e) - 8388608.f, f1 = byte_float(sl1[tw], e) - 8388608.f;
          su[0] = fmaf(f0, part[0], su[0]), su[1] = fmaf(f0, part[1], su[1]);
          su[2] = fmaf(f1, part[2], su[2]), su[3] = fmaf(f1, part[3], su[3]);
        }
      }
    }
    // sum_is min_is * (sum of x over sub-block is): the MMA over sub-blocks; this lane's slots are
    // sub-blocks 2t, 2t + 1, 2t + 8, 2t + 9, the word t of each row's sixteen bytes, high nibbles
    const uint32_t m0 = ((t == 0 ? h0.x : t == 1 ? h0.y : t == 2 ? h0.z : h0.w) >> 4) & 0x0f0f0f0fu;
    const uint32_t m1 = ((t == 0 ? h1.x : t == 1 ? h1.y : t == 2 ? h1.z : h1.w) >> 4) & 0x0f0f0f0fu;
    const uint4 bs = lds128(xu + kXSums + (uint32_t)lane * 16u);
    float cm[4];
    const uint32_t a0 = byte_pair(m0, 0x4140u), a1 = byte_pair(m1, 0x4140u);
    const uint32_t a2 = byte_pair(m0, 0x4342u), a3 = byte_pair(m1, 0x4342u);
    mma16816_first(cm, a0, a1, a2, a3, bs.x, bs.y);
    mma16816(cm, a0, a1, a2, a3, bs.z, bs.w);
    const uint32_t dd = lds32(tile + 1280u + (uint32_t)g * 4u), mm = lds32(tile + 1312u + (uint32_t)g * 4u);
    const float d0 = half_bits_to_float(dd & 0xffffu) * 16777216.f, d1 = half_bits_to_float(dd >> 16) * 16777216.f;
    const float n0 = -half_bits_to_float(mm & 0xffffu), n1 = -half_bits_to_float(mm >> 16);
    acc[0] = fmaf(d0, su[0], fmaf(n0, cm[0], acc[0]));
    acc[1] = fmaf(d0, su[1], fmaf(n0, cm[1], acc[1]));
    acc[2] = fmaf(d1, su[2], fmaf(n1, cm[2], acc[2]));
    acc[3] = fmaf(d1, su[3], fmaf(n1, cm[3], acc[3]));
  }
};

}  // namespace ishi
