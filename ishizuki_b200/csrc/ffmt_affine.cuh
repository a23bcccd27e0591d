// MLX affine group-quantized packs (4 or 2 bits, fp16 or bf16 scales) for the warp-level kernel.
//
// Layout of the source (reference: Sources/IshizukiKit/Core/VerifyMatmul.swift:282-287 and
// Sources/IshizukiKit/Quantize/WeightedAffineQuantizer.swift:142-161): row n is K*bits/32
// little-endian uint32 words, code i of a word at bit i*bits; w = float(code) * scale + bias with
// one (scale, bias) pair per group of GS inputs.
//
// The product is factored per group as the reference's codes kernel does
// (VerifyMatmul.swift:123-128): y += s_g * sum_k code_k x_k + b_g * sum_k x_k. Codes masked in
// place are fp16 bit patterns of code * 2^-24 times the power of two of their bit position; that
// extra power of two is taken out on the activation side, where x is staged divided by it (exact
// unless |x| is tiny, where it costs at most half a unit in the last place of an fp16
// subnormal). The second sum uses fp32 group sums of x staged beside the fragments.
//
// Fragment mapping (m16n8k16; lane g = lane / 4, t = lane % 4 holds weight rows g and g + 8): of
// every four consecutive words ("quad" q) lane t owns word 4q + t of both rows. One word yields
// the A registers of 8 / BITS ... k-steps: with mask m (the m-th code of each byte pair),
//   4 bits: k-step (q, m), m < 2:  a0 = codes (m, m + 4), a2 = codes (m + 2, m + 6) of the word
//   2 bits: k-step (q, m), m < 4:  a0 = codes (m, m + 8), a2 = codes (m + 4, m + 12)
// and x is staged in exactly that order, scaled by 2^-(BITS * m).
//
// Tile (16 rows x 256 k): BITS pieces of 512 bytes, piece j = [lane][row g: words of quads 2j and
// 2j + 1; row g + 8: the same], then per row the unit's scales followed by its biases.
#pragma once
#include <cuda_bf16.h>

#include "ishi_fragstream.cuh"

namespace ishi {

template <int BITS, int GS, bool BF16>
struct FragAffine {
  static_assert(BITS == 4 || BITS == 2, "4- and 2-bit codes");
  static_assert(GS == 32 || GS == 64 || GS == 128, "group sizes of the reference");
  static_assert(BITS == 4 || GS >= 64, "a 2-bit k-step spans 64 inputs");
  static constexpr int kGroups = 256 / GS;           // per unit
  static constexpr int kQuads = 2 * BITS;            // word quads per unit: 8 (32 words) or 4 (16 words)
  static constexpr int kMasks = 8 / BITS;            // k-steps per quad: 2 or 4
  static constexpr int kQuadK = 256 / kQuads;        // inputs a quad covers: 32 or 64
  static constexpr int kHeader = BITS * 512;         // offset of the scales and biases
  static constexpr int kRowHeader = 4 * kGroups;     // bytes per row there
  static constexpr int kTileBytes = kHeader + 16 * kRowHeader;
  static constexpr int kSums = 4096;                 // offset of the group sums of x: [group][activation row] fp32
  static constexpr int kExtraBytes = 0;  // shared memory per CTA beyond the per-unit staging
  static constexpr bool kRowMode = true;  // MODE 1: one activation row on CUDA cores
  static constexpr int kXBytes = 4096 + (32 * kGroups > 128 ? 32 * kGroups : 128);

  static __device__ __forceinline__ uint16_t tile_halfword(const FragSrc &s, long long p, int u, int hw) {
    if (hw < kHeader / 2) {
      const int c = hw >> 8, lane = (hw & 255) >> 3, h = hw & 7;
      const int g = lane >> 2, t = lane & 3;
      const long long row = p * kFragRows + g + 8 * (h >> 2);
      if (row >= s.N) return 0;
      const int q = 2 * c + ((h & 3) >> 1);
      const long long word = (long long)u * (8 * BITS) + 4 * q + t;
      long long local;
      const int seg = frag_segment(s, row, &local);
      return *reinterpret_cast<const uint16_t *>(s.w[seg] + local * s.w_row_bytes + word * 4 + 2 * (h & 1));
    }
    const int idx = hw - kHeader / 2;
    const long long row = p * kFragRows + idx / (2 * kGroups);
    const int j = idx % (2 * kGroups);
    if (row >= s.N) return 0;
    long long local;
    const int seg = frag_segment(s, row, &local);
    const uint8_t *base = j < kGroups ? s.scales[seg] : s.biases[seg];
    return *reinterpret_cast<const uint16_t *>(base + local * s.s_row_bytes + ((long long)u * kGroups + (j % kGroups)) * 2);
  }

  // x * 2^-e on both halves (exact power-of-two scaling)
  template <int E>
  static __device__ __forceinline__ uint32_t scale_down(uint32_t v) {
    if (E == 0) return v;
    const __half2 f = __float2half2_rn(1.0f / (float)(1 << E));
    const __half2 r = __hmul2(*reinterpret_cast<const __half2 *>(&v), f);
    return *reinterpret_cast<const uint32_t *>(&r);
  }

  // nothing to set up ahead of the dependency wait
  static __device__ __forceinline__ void before_wait(const FragArgs &, uint32_t) {}

  // Activations of the CTA's column range into fragment order. A warp task is (unit, activation
  // row): lane l loads the eight values k = 8l .. 8l + 7. The fragment of k-step st = kMasks * q + m
  // sits at st * 256 + ((g ^ (q & 3)) * 4 + t) * 8: the xor spreads a store's quads over the banks,
  // and a k-step's 32 lanes still read one 256-byte run.
  // after_loads() runs once, when the first batch of loads is in flight and before their values are
  // used (the kernel issues its first weight copies there, behind the activations).
  template <class F>
  static __device__ __forceinline__ void stage_x(const FragArgs &a, uint32_t xfrag, int ub0, int uc, F &&after_loads) {
    if (BITS == 2 && GS == 128 && a.rot_block == 128 && !a.rot_signs) {
      stage_x_rot128(a, xfrag, ub0, uc, after_loads);
      return;
    }
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
        const int g = i & 7;
        if (a.rot_block)
          v[e] = frag_rotate8(v[e], a.rot_block,
                              a.rot_signs ? a.rot_signs + (long long)(ub0 + (i >> 3)) * 256 + lane * 8 : nullptr, lane);
        const uint32_t base = xfrag + (uint32_t)(i >> 3) * kXBytes;
        // halves of v: x0 x1 | x2 x3 | x4 x5 | x6 x7
        if (BITS == 4) {
          // the lane holds word l: quad q = l / 4, t = l % 4; k-step m pairs (x_m, x_m+4), (x_m+2, x_m+6)
          const int q = lane >> 2, t = lane & 3;
          const uint32_t dst = base + (uint32_t)(2 * q) * 256u + (uint32_t)(((g ^ (q & 3)) * 4 + t) * 8);
          sts64(dst, prmt(v[e].x, v[e].z, 0x5410u), prmt(v[e].y, v[e].w, 0x5410u));
          sts64(dst + 256u, scale_down<4>(prmt(v[e].x, v[e].z, 0x7632u)), scale_down<4>(prmt(v[e].y, v[e].w, 0x7632u)));
        } else {
          // the lane holds half of word l / 2 (codes 0..7 when l is even, 8..15 when odd): quad
          // q = l / 8, t = (l / 2) % 4. k-step m pairs (x_m, x_m+8), (x_m+4, x_m+12): the even lane
          // builds m = 0, 1 and the odd lane m = 2, 3, each with the other's half of the word.
          const uint32_t ox = __shfl_xor_sync(0xffffffffu, v[e].x, 1), oy = __shfl_xor_sync(0xffffffffu, v[e].y, 1);
          const uint32_t oz = __shfl_xor_sync(0xffffffffu, v[e].z, 1), ow = __shfl_xor_sync(0xffffffffu, v[e].w, 1);
          const bool odd = lane & 1;
          // lo = codes 0..7 of the word, hi = codes 8..15
          const uint32_t lx = odd ? ox : v[e].x, ly = odd ? oy : v[e].y, lz = odd ? oz : v[e].z, lw = odd ? ow : v[e].w;
          const uint32_t hx = odd ? v[e].x : ox, hy = odd ? v[e].y : oy, hz = odd ? v[e].z : oz, hw = odd ? v[e].w : ow;
          const int q = lane >> 3, t = (lane >> 1) & 3;
          const uint32_t dst = base + (uint32_t)(4 * q + (odd ? 2 : 0)) * 256u + (uint32_t)(((g ^ (q & 3)) * 4 + t) * 8);
          // m = 0 / 2: (lo_m, hi_m), (lo_m+4, hi_m+4) with lo_0 = lx.lo, lo_2 = ly.lo, lo_4 = lz.lo, lo_6 = lw.lo
          const uint32_t ea = odd ? ly : lx, eb = odd ? hy : hx, ec = odd ? lw : lz, ed = odd ? hw : hz;
          if (odd) {
            sts64(dst, scale_down<4>(prmt(ea, eb, 0x5410u)), scale_down<4>(prmt(ec, ed, 0x5410u)));
            sts64(dst + 256u, scale_down<6>(prmt(ea, eb, 0x7632u)), scale_down<6>(prmt(ec, ed, 0x7632u)));
          } else {
            sts64(dst, prmt(ea, eb, 0x5410u), prmt(ec, ed, 0x5410u));
            sts64(dst + 256u, scale_down<2>(prmt(ea, eb, 0x7632u)), scale_down<2>(prmt(ec, ed, 0x7632u)));
          }
        }
        // fp32 sums of x over the groups (GS / 8 lanes each), for the bias term
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].y));
        const float2 f2 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].z));
        const float2 f3 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].w));
        float s = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
#pragma unroll
        for (int d = 1; d < GS / 8; d *= 2) s += __shfl_xor_sync(0xffffffffu, s, d);
        if ((lane & (GS / 8 - 1)) == 0)
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(base + kSums + (uint32_t)((lane / (GS / 8)) * 8 + g) * 4u), "f"(s)
                       : "memory");
      }
    }
  }

  // +1 or -1 in fp16 by the parity of v
  static __device__ __forceinline__ uint32_t sign_half(int v) { return 0x3c00u | ((uint32_t)(__popc(v) & 1) << 15); }
  static __device__ __forceinline__ uint32_t pack_rn(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
  }

  // The 2-bit staging with the block Hadamard rotation of 128 (no sign vector) on the tensor
  // cores. With k = 8 i + j inside a block (i < 16, j < 8) the natural-order transform factors as
  // H128 = H16 (x) H8, so the rotated block, seen as the matrix Y[j'][i'], is H8 * X^T * H16:
  //   stage 1: Z[j'][i] = sum_j H8[j'][j] x[8 i + j]. One m16n8k16 takes both blocks of a unit:
  //     A = [H8 0; 0 H8] (rows j' of the first block, then of the second), B rows k = j of the
  //     first block then of the second, columns i of one half (eight of the sixteen): lane
  //     (g, t) supplies the 32-bit word g * 4 + t of that half, a coalesced load.
  //   stage 2: Y[j'][i'] = sum_i Z[j'][i] H16[i][i'], A = Z of both blocks (the fp32 sums of
  //     stage 1 as fp16 high and low parts, two MMAs, so nothing is lost to the fp16 operand),
  //     B = H16, columns i' of one half.
  // The fp32 result times 1 / sqrt(128) is rounded to fp16 as the butterfly's is; the two agree
  // to fp32 rounding. Lane (g, t) ends up with the values k' = 16 (4 h + t) + g and + 8 of each
  // block: the codes g and g + 8 of the block's word 4 h + t, which are one B register of the
  // product's k-step (quad 2 block + h, mask g % 4), low register when g < 4.
  template <class F>
  static __device__ __forceinline__ void stage_x_rot128(const FragArgs &a, uint32_t xfrag, int ub0, int uc, F &&after_loads) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tasks = uc * 8;
    constexpr int kBatch = 8;
    const uint32_t h8 = sign_half(g & (2 * t)) | (sign_half(g & (2 * t + 1)) << 16);
    uint32_t h16[2][2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = 8 * h + g;
      h16[h][0] = sign_half(n & (2 * t)) | (sign_half(n & (2 * t + 1)) << 16);
      h16[h][1] = sign_half(n & (2 * t + 8)) | (sign_half(n & (2 * t + 9)) << 16);
    }
    const int m = g & 3;
    const uint32_t down1 = (uint32_t)(15 - 2 * m) << 10;  // 2^-(2 m) in fp16
    const uint32_t down = down1 | (down1 << 16);
    const float scale = 1.0f / sqrtf(128.f);
    const uint32_t *xl = reinterpret_cast<const uint32_t *>(a.x + (long long)ub0 * 256) + lane;
    const long long row_words = a.K >> 1;
    if (warp >= tasks) after_loads();
    for (int i0 = warp; i0 < tasks; i0 += nw * kBatch) {
      uint32_t v[kBatch][4];  // [block * 2 + half]
#pragma unroll
      for (int e = 0; e < kBatch; ++e) {
        const int i = i0 + e * nw;
        const bool live = i < tasks && (i & 7) < a.M;
        const uint32_t *src = xl + (long long)(i & 7) * row_words + (i >> 3) * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) v[e][c] = live ? __ldg(src + 32 * c) : 0u;
      }
      if (i0 == warp) after_loads();
#pragma unroll
      for (int e = 0; e < kBatch; ++e) {
        const int i = i0 + e * nw;
        if (i >= tasks) break;
        const int r = i & 7;
        const uint32_t base = xfrag + (uint32_t)(i >> 3) * kXBytes;
        uint32_t zh[4], zl[4];  // stage 2's A registers: (block 0, half 0), (block 1, half 0), (block 0, half 1), (block 1, half 1)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float z[4];
          mma16816_first(z, h8, 0u, 0u, h8, v[e][h], v[e][2 + h]);
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            const uint32_t hi = pack_rn(z[2 * b], z[2 * b + 1]);
            const float2 hf = __half22float2(*reinterpret_cast<const __half2 *>(&hi));
            zh[2 * h + b] = hi;
            zl[2 * h + b] = pack_rn(z[2 * b] - hf.x, z[2 * b + 1] - hf.y);
          }
        }
        float sum[2] = {0.f, 0.f};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float y[4];
          mma16816_first(y, zh[0], zh[1], zh[2], zh[3], h16[h][0], h16[h][1]);
          mma16816(y, zl[0], zl[1], zl[2], zl[3], h16[h][0], h16[h][1]);
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            const uint32_t pr = pack_rn(__fmul_rn(y[2 * b], scale), __fmul_rn(y[2 * b + 1], scale));
            const float2 pf = __half22float2(*reinterpret_cast<const __half2 *>(&pr));
            sum[b] += pf.x + pf.y;
            const __half2 sc = __hmul2(*reinterpret_cast<const __half2 *>(&pr), *reinterpret_cast<const __half2 *>(&down));
            const int q = 2 * b + h;
            sts32(base + (uint32_t)(4 * q + m) * 256u + (uint32_t)(((r ^ q) * 4 + t) * 8 + (g >> 2) * 4),
                  *reinterpret_cast<const uint32_t *>(&sc));
          }
        }
        // fp32 sums of the rounded values over each block (the group of the bias term): the lower
        // half warp collects the first block, the upper half the second
        const bool up = lane & 16;
        float keep = up ? sum[1] : sum[0];
        keep += __shfl_xor_sync(0xffffffffu, up ? sum[0] : sum[1], 16);
#pragma unroll
        for (int d = 8; d; d >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, d);
        if ((lane & 15) == 0)
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(base + kSums + (uint32_t)((lane >> 4) * 8 + r) * 4u), "f"(keep) : "memory");
      }
    }
  }

  static __device__ __forceinline__ float param(uint32_t pair, int hi) {
    if (BF16) return hi ? __uint_as_float(pair & 0xffff0000u) : __uint_as_float(pair << 16);
    return half_bits_to_float(hi ? pair >> 16 : pair & 0xffffu);
  }
  static __device__ __forceinline__ float half_lo(uint32_t pair) { return __half2float(__ushort_as_half((unsigned short)(pair & 0xffffu))); }
  static __device__ __forceinline__ float half_hi(uint32_t pair) { return __half2float(__ushort_as_half((unsigned short)(pair >> 16))); }

  // One tile against the activations of its unit. acc: the warp's C fragment (MODE 0) or this
  // lane's partial dot products of rows g (acc[0]) and g + 8 (acc[2]) (MODE 1).
  template <int MODE>
  static __device__ __forceinline__ void unit(float (&acc)[4], const FragArgs &a, uint32_t tile, uint32_t xbase, int uq,
                                              int g, int t, int lane) {
    const uint32_t xu = xbase + (uint32_t)uq * kXBytes;
    // scales and biases of the two rows: kGroups halfwords of each, packed in pairs
    uint32_t hdr0[kRowHeader / 4], hdr1[kRowHeader / 4];
    if (kRowHeader == 8) {
      const uint2 p0 = lds64(tile + kHeader + (uint32_t)g * 8u), p1 = lds64(tile + kHeader + (uint32_t)(g + 8) * 8u);
      hdr0[0] = p0.x, hdr0[1] = p0.y, hdr1[0] = p1.x, hdr1[1] = p1.y;
    } else {
#pragma unroll
      for (int i = 0; i < kRowHeader / 16; ++i) {
        const uint4 p0 = lds128(tile + kHeader + (uint32_t)g * kRowHeader + 16u * i);
        const uint4 p1 = lds128(tile + kHeader + (uint32_t)(g + 8) * kRowHeader + 16u * i);
        hdr0[4 * i] = p0.x, hdr0[4 * i + 1] = p0.y, hdr0[4 * i + 2] = p0.z, hdr0[4 * i + 3] = p0.w;
        hdr1[4 * i] = p1.x, hdr1[4 * i + 1] = p1.y, hdr1[4 * i + 2] = p1.z, hdr1[4 * i + 3] = p1.w;
      }
    }
    const uint32_t xl = xu + (uint32_t)(MODE == 0 ? lane : t) * 8u;  // single row: the fragments of activation row 0
    float part[4];

#pragma unroll
    for (int j = 0; j < BITS; ++j) {
      const uint4 w = lds128(tile + (uint32_t)j * 512u + (uint32_t)lane * 16u);  // row g: w.x, w.y; row g + 8: w.z, w.w
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const int q = 2 * j + s;
        const uint32_t x0 = s ? w.y : w.x, x1 = s ? w.w : w.z;
        const uint32_t y0 = x0 >> 8, y1 = x1 >> 8;
        const uint32_t xq = xl ^ (uint32_t)((q & 3) << 5);  // the quad's staging swizzle
#pragma unroll
        for (int m = 0; m < kMasks; ++m) {
          const uint32_t mask = (BITS == 4 ? 0x000f000fu : 0x00030003u) << (BITS * m);
          const uint32_t a0 = x0 & mask, a1 = x1 & mask, a2 = y0 & mask, a3 = y1 & mask;
          const uint2 b = lds64(xq + (uint32_t)(kMasks * q + m) * 256u);
          const bool first = (q * kQuadK) % GS == 0 && m == 0;  // first k-step of a group
          if (MODE == 0) {
            if (first) mma16816_first(part, a0, a1, a2, a3, b.x, b.y);
            else mma16816(part, a0, a1, a2, a3, b.x, b.y);
          } else {
            if (first) part[0] = part[1] = part[2] = part[3] = 0.f;
            part[0] = fmaf(half_lo(a0), half_lo(b.x), part[0]);
            part[0] = fmaf(half_hi(a0), half_hi(b.x), part[0]);
            part[0] = fmaf(half_lo(a2), half_lo(b.y), part[0]);
            part[0] = fmaf(half_hi(a2), half_hi(b.y), part[0]);
            part[2] = fmaf(half_lo(a1), half_lo(b.x), part[2]);
            part[2] = fmaf(half_hi(a1), half_hi(b.x), part[2]);
            part[2] = fmaf(half_lo(a3), half_lo(b.y), part[2]);
            part[2] = fmaf(half_hi(a3), half_hi(b.y), part[2]);
          }
        }
        if (((q + 1) * kQuadK) % GS == 0) {
          // the group is complete: scale its code sum, add bias times the group's sum of x
          const int grp = (q * kQuadK) / GS;
          const float s0 = param(hdr0[grp >> 1], grp & 1) * 16777216.f;
          const float s1 = param(hdr1[grp >> 1], grp & 1) * 16777216.f;
          const float b0 = param(hdr0[(kGroups + grp) >> 1], (kGroups + grp) & 1);
          const float b1 = param(hdr1[(kGroups + grp) >> 1], (kGroups + grp) & 1);
          if (MODE == 0) {
            const float2 xs = lds64f(xu + kSums + (uint32_t)(grp * 8 + 2 * t) * 4u);
            acc[0] += s0 * part[0] + b0 * xs.x;
            acc[1] += s0 * part[1] + b0 * xs.y;
            acc[2] += s1 * part[2] + b1 * xs.x;
            acc[3] += s1 * part[3] + b1 * xs.y;
          } else {
            // the bias term enters once per row: lane t = 0 adds it
            const float xs = t == 0 ? lds32f(xu + kSums + (uint32_t)(grp * 8) * 4u) : 0.f;
            acc[0] += s0 * part[0] + b0 * xs;
            acc[2] += s1 * part[2] + b1 * xs;
          }
        }
      }
    }
  }
};

}  // namespace ishi
