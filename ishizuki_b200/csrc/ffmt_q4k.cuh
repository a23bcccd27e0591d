// GGUF Q4_K for the warp-level kernel (mma.sync fragments, or CUDA-core FMA for one row).
//
// Block layout (144 bytes per 256 weights; reference: Sources/IshizukiKit/Core/GGMLDequant.swift
// :187-220 and the kernel body at Sources/IshizukiKit/Core/GGMLKernels.swift:586-603):
//   d f16 @0, dmin f16 @2, twelve bytes of 6-bit (scale, min) pairs @4, 128 nibble bytes @16.
//   Byte l of 32-byte chunk j holds weight 64j + l (low nibble, sub-block 2j) and weight
//   64j + 32 + l (high nibble, sub-block 2j + 1);  w = d * sc * q - dmin * m.
//
// The product is factored as the reference's matvec does (GGMLKernels.swift:432-440):
//   y += d * sum_sb sc_sb * (sum_k q_k x_k) - dmin * sum_sb m_sb * (sum_k x_k),
// with the integer sub-block scale folded into the fragment before the MMA: q * sc <= 945 is an
// exact fp16 number, so a whole tile accumulates in the tensor core and only d and dmin remain
// for fp32. A nibble masked in place is the bit pattern of the fp16 number q * 2^-24 (low) or
// q * 2^-20 (high); the low ones take their scale by an integer multiply on the packed pair
// (q * sc < 1024 stays a subnormal bit pattern), the high ones by a half2 multiply.
//
// Fragment mapping (m16n8k16; lane g = lane / 4, t = lane % 4 holds weight rows g and g + 8).
// Lane t owns chunk t of both rows, i.e. exactly sub-blocks 2t (low nibbles) and 2t + 1 (high
// nibbles): a lane unpacks two scales and two minima per row instead of all sixteen, and the
// minima it holds are the ones its slots of the minimum-term MMA need. One MMA therefore mixes
// four sub-blocks (one per t), which is why the scales go into the fragments. A k-step is
// (piece jj, word s, half h): lane t works on bytes 8j .. 8j + 7 of its chunk with
// j = (jj + t) % 4 (the rotation keeps the four lanes of a row off each other's shared-memory
// banks when they read the activations), word s of them, low or high nibbles:
// k = 64t + 32h + 8j + 4s + {0, 1, 2, 3}. Inside a stored word the bytes are in the order
// (k0, k0 + 2, k0 + 1, k0 + 3), so that the masked word is the A register of slots (2t, 2t + 1) and
// the word shifted by eight bits that of slots (2t + 8, 2t + 9), both in natural k order: the
// activations are used as they lie in memory.
//
// Tile (16 rows x 256 k, 2368 bytes): piece jj = [lane][row g: 8 bytes, row g + 8: 8 bytes] for
// jj = 0..3; then per row and t one word with the bytes m[2t], sc[2t], m[2t+1], sc[2t+1] (the
// six-bit fields of the block's twelve packed bytes, one per byte: a lane's scales and minima then
// come out with one byte permute or mask each; 64 bytes more than the 2304 of the blocks); then d
// and dmin of every row.
//
// Activations of a unit in shared memory: eight rows of 256 fp16 as they lie in x, 576 bytes
// apart (rows g and g + 1 then sit 64 bytes apart modulo the 128 bytes of a bank sweep), copied by
// the bulk copy engine; then the sub-block sums of x for the minimum term.
#pragma once
#include "ishi_fragstream.cuh"

namespace ishi {

struct FragQ4K {
  static constexpr int kTileBytes = 2048 + 16 * 16 + 16 * 4;
  static constexpr int kExtraBytes = 0;  // shared memory per CTA beyond the per-unit staging
  static constexpr bool kRowMode = true;  // MODE 1: one activation row on CUDA cores
  static constexpr int kSumBytes = 384;  // per unit: sub-block sums as fp16 hi / lo pairs, [lane][8 bytes], then
                                         // the fp32 sub-block sums of row 0 (single-row kernel) @256
  // shared memory the kernel sets aside per unit of the column range: eight rows of 512 bytes, the
  // sums, and a share of the rows' 64-byte skew (8 * 64 <= 512 for any range of one unit or more)
  static constexpr int kXBytes = 8 * 512 + kSumBytes + 512;

  // ggml's get_scale_min_k4 on the twelve packed bytes of a block
  static __device__ __forceinline__ void scale_min(const uint8_t *q, int j, uint32_t *sc, uint32_t *m) {
    if (j < 4) {
      *sc = q[j] & 63u;
      *m = q[j + 4] & 63u;
    } else {
      *sc = (q[j + 4] & 0xfu) | ((uint32_t)(q[j - 4] >> 6) << 4);
      *m = (uint32_t)(q[j + 4] >> 4) | ((uint32_t)(q[j] >> 6) << 4);
    }
  }

  static __device__ __forceinline__ uint8_t tile_byte(const FragSrc &s, long long p, int u, int b) {
    if (b < 2048) {
      const int jj = b >> 9, lane = (b & 511) >> 4, i = b & 15;
      const int g = lane >> 2, t = lane & 3;
      const long long row = p * kFragRows + g + 8 * (i >> 3);
      if (row >= s.N) return 0;
      const int j = jj ^ t, word = (i & 7) >> 2, pos = i & 3;
      const int k = pos == 0 ? 0 : pos == 1 ? 2 : pos == 2 ? 1 : 3;  // stored order (k0, k0 + 2, k0 + 1, k0 + 3)
      long long local;
      const int seg = frag_segment(s, row, &local);
      return s.w[seg][local * s.w_row_bytes + (long long)u * 144 + 16 + 32 * t + 8 * j + 4 * word + k];
    }
    const int idx = b - 2048;
    if (idx < 256) {
      const long long row = p * kFragRows + (idx >> 4);
      if (row >= s.N) return 0;
      long long local;
      const int seg = frag_segment(s, row, &local);
      const uint8_t *blk = s.w[seg] + local * s.w_row_bytes + (long long)u * 144;
      const int t = (idx >> 2) & 3, byte = idx & 3;
      uint32_t sc, m;
      scale_min(blk + 4, 2 * t + (byte >> 1), &sc, &m);
      return (uint8_t)((byte & 1) ? sc : m);
    }
    const long long row = p * kFragRows + ((idx - 256) >> 2);
    if (row >= s.N) return 0;
    long long local;
    const int seg = frag_segment(s, row, &local);
    return s.w[seg][local * s.w_row_bytes + (long long)u * 144 + (idx & 3)];
  }

  static __device__ __forceinline__ uint16_t tile_halfword(const FragSrc &s, long long p, int u, int hw) {
    return (uint16_t)(tile_byte(s, p, u, 2 * hw) | ((uint32_t)tile_byte(s, p, u, 2 * hw + 1) << 8));
  }

  // Activations of the CTA's column range. A warp task is (unit, activation row): lane l loads
  // k = 8l .. 8l + 7 of it, stores them as they lie in x (rows past M as zeros) and the warp adds up
  // every sub-block for the minimum term. after_loads() runs once, when the first batch of loads is
  // in flight. Q4_K has no input rotation.
  static __device__ __forceinline__ uint32_t row_stride(const FragArgs &a) { return (uint32_t)a.umax * 512u + 64u; }

  // nothing to set up ahead of the dependency wait
  static __device__ __forceinline__ void before_wait(const FragArgs &, uint32_t) {}

  template <class F>
  static __device__ __forceinline__ void stage_x(const FragArgs &a, uint32_t xfrag, int ub0, int uc, F &&after_loads) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const uint32_t R = row_stride(a), sums = xfrag + 8u * R;
    const int tasks = uc * 8, jj = lane >> 3;
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
        sts128u(xfrag + (uint32_t)r * R + (uint32_t)u * 512u + (uint32_t)lane * 16u, v[e]);
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].y));
        const float2 f2 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].z));
        const float2 f3 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].w));
        float s = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        const float o = __shfl_xor_sync(0xffffffffu, s, 4);
        const uint32_t base = sums + (uint32_t)u * kSumBytes;
        if ((lane & 7) == 0) {
          // sub-blocks 2t' and 2t' + 1 (t' = lane / 8) of activation row r, as fp16 hi + lo: the B
          // fragment of the minimum-term MMA, whose k index runs over sub-blocks
          const __half h0 = __float2half_rn(s), h1 = __float2half_rn(o);
          const __half l0 = __float2half_rn(s - __half2float(h0)), l1 = __float2half_rn(o - __half2float(h1));
          sts64(base + (uint32_t)(r * 4 + jj) * 8u, (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16),
                (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16));
        }
        if (r == 0 && (lane & 3) == 0)  // fp32 sums of activation row 0 (the single-row kernel's minimum term)
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(base + 256u + (uint32_t)(lane >> 2) * 4u), "f"(s) : "memory");
      }
    }
  }

  static __device__ __forceinline__ float half_lo(uint32_t pair) { return __half2float(__ushort_as_half((unsigned short)(pair & 0xffffu))); }
  static __device__ __forceinline__ float half_hi(uint32_t pair) { return __half2float(__ushort_as_half((unsigned short)(pair >> 16))); }

  // One tile against the activations of its unit. acc: the warp's C fragment (MODE 0) or this
  // lane's partial dot products of rows g (acc[0]) and g + 8 (acc[2]) (MODE 1).
  template <int MODE>
  static __device__ __forceinline__ void unit(float (&acc)[4], const FragArgs &a, uint32_t tile, uint32_t xbase, int uq,
                                              int g, int t, int lane) {
    // this lane's sub-blocks 2t, 2t + 1 of rows g and g + 8: bytes m_lo, sc_lo, m_hi, sc_hi
    const uint32_t v0 = lds32(tile + 2048u + (uint32_t)lane * 4u), v1 = lds32(tile + 2048u + 128u + (uint32_t)lane * 4u);
    const uint32_t dd0 = lds32(tile + 2304u + (uint32_t)g * 4u), dd1 = lds32(tile + 2304u + 32u + (uint32_t)g * 4u);
    // low sub-block: the scale as an integer; high sub-block: sc / 16 as a half2 pair (the bits of
    // 64 + sc / 16, minus 64), so that both products come out in units of 2^-24
    const uint32_t sl0 = prmt(v0, 0u, 0x4441u), sl1 = prmt(v1, 0u, 0x4441u);
    const __half2 k64 = __float2half2_rn(64.f);
    const uint32_t sh0p = prmt(v0, 0x54545454u, 0x4343u), sh1p = prmt(v1, 0x54545454u, 0x4343u);
    const __half2 sh0 = __hsub2(*reinterpret_cast<const __half2 *>(&sh0p), k64);
    const __half2 sh1 = __hsub2(*reinterpret_cast<const __half2 *>(&sh1p), k64);
    // the lane's activation row: its own fragment column (MODE 0) or row 0 (MODE 1), chunk t, and
    // piece t of it (bits 4 and 5 of the address, which the pieces' rotation then flips)
    const uint32_t R = row_stride(a);
    const uint32_t xrow = xbase + (uint32_t)(MODE == 0 ? g : 0) * R + (uint32_t)t * 144u + (uint32_t)uq * 512u;
    const uint32_t xsum = xbase + 8u * R + (uint32_t)uq * kSumBytes;

    float c[4] = {0.f, 0.f, 0.f, 0.f};  // one MMA chain over the whole tile
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const uint4 w = lds128(tile + (uint32_t)jj * 512u + (uint32_t)lane * 16u);  // row g: w.x, w.y; row g + 8: w.z, w.w
      const uint32_t xj = xrow ^ (uint32_t)(jj << 4);        // piece jj ^ t of the chunk
      const uint4 blo = lds128(xj), bhi = lds128(xj + 64u);  // k-steps (s = 0, 1) of the low / high sub-block
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const uint32_t x0 = s ? w.y : w.x, x1 = s ? w.w : w.z;
        const uint32_t y0 = x0 >> 8, y1 = x1 >> 8;
        const uint32_t bl0 = s ? blo.z : blo.x, bl1 = s ? blo.w : blo.y;
        const uint32_t bh0 = s ? bhi.z : bhi.x, bh1 = s ? bhi.w : bhi.y;
        // low nibbles: q * sc as an integer in each half (a subnormal fp16 bit pattern, x 2^-24)
        const uint32_t a0 = (x0 & 0x000f000fu) * sl0, a1 = (x1 & 0x000f000fu) * sl1;
        const uint32_t a2 = (y0 & 0x000f000fu) * sl0, a3 = (y1 & 0x000f000fu) * sl1;
        // high nibbles: (q * 2^-20) * (sc / 16) by a half2 multiply (exact: q * sc < 1024, still subnormal)
        const uint32_t m0 = x0 & 0x00f000f0u, m1 = x1 & 0x00f000f0u, m2 = y0 & 0x00f000f0u, m3 = y1 & 0x00f000f0u;
        const __half2 c0 = __hmul2(*reinterpret_cast<const __half2 *>(&m0), sh0);
        const __half2 c1 = __hmul2(*reinterpret_cast<const __half2 *>(&m1), sh1);
        const __half2 c2 = __hmul2(*reinterpret_cast<const __half2 *>(&m2), sh0);
        const __half2 c3 = __hmul2(*reinterpret_cast<const __half2 *>(&m3), sh1);
        const uint32_t e0 = *reinterpret_cast<const uint32_t *>(&c0), e1 = *reinterpret_cast<const uint32_t *>(&c1);
        const uint32_t e2 = *reinterpret_cast<const uint32_t *>(&c2), e3 = *reinterpret_cast<const uint32_t *>(&c3);
        if (MODE == 0) {
          if (jj == 0 && s == 0)
            mma16816_first(c, a0, a1, a2, a3, bl0, bl1);
          else
            mma16816(c, a0, a1, a2, a3, bl0, bl1);
          mma16816(c, e0, e1, e2, e3, bh0, bh1);
        } else {
          c[0] = fmaf(half_lo(a0), half_lo(bl0), c[0]);
          c[0] = fmaf(half_hi(a0), half_hi(bl0), c[0]);
          c[0] = fmaf(half_lo(a2), half_lo(bl1), c[0]);
          c[0] = fmaf(half_hi(a2), half_hi(bl1), c[0]);
          c[2] = fmaf(half_lo(a1), half_lo(bl0), c[2]);
          c[2] = fmaf(half_hi(a1), half_hi(bl0), c[2]);
          c[2] = fmaf(half_lo(a3), half_lo(bl1), c[2]);
          c[2] = fmaf(half_hi(a3), half_hi(bl1), c[2]);
          c[1] = fmaf(half_lo(e0), half_lo(bh0), c[1]);
          c[1] = fmaf(half_hi(e0), half_hi(bh0), c[1]);
          c[1] = fmaf(half_lo(e2), half_lo(bh1), c[1]);
          c[1] = fmaf(half_hi(e2), half_hi(bh1), c[1]);
          c[3] = fmaf(half_lo(e1), half_lo(bh0), c[3]);
          c[3] = fmaf(half_hi(e1), half_hi(bh0), c[3]);
          c[3] = fmaf(half_lo(e3), half_lo(bh1), c[3]);
          c[3] = fmaf(half_hi(e3), half_hi(bh1), c[3]);
        }
      }
    }

    const float d0 = half_bits_to_float(dd0 & 0xffffu) * 16777216.f, d1 = half_bits_to_float(dd1 & 0xffffu) * 16777216.f;
    const float n0 = half_bits_to_float(dd0 >> 16), n1 = half_bits_to_float(dd1 >> 16);
    if (MODE == 0) {
      // minimum term: one MMA whose k index runs over sub-blocks (hi parts in k 0..7, lo in 8..15);
      // this lane's slots are sub-blocks 2t and 2t + 1, exactly the minima it holds
      const uint32_t ma = v0 & 0x00ff00ffu, mb = v1 & 0x00ff00ffu;
      const uint2 xs = lds64(xsum + (uint32_t)lane * 8u);
      float cm[4];
      mma16816_first(cm, ma, mb, ma, mb, xs.x, xs.y);
      const float m0 = n0 * -16777216.f, m1 = n1 * -16777216.f;
      acc[0] = fmaf(d0, c[0], fmaf(m0, cm[0], acc[0]));
      acc[1] = fmaf(d0, c[1], fmaf(m0, cm[1], acc[1]));
      acc[2] = fmaf(d1, c[2], fmaf(m1, cm[2], acc[2]));
      acc[3] = fmaf(d1, c[3], fmaf(m1, cm[3], acc[3]));
    } else {
      // the lane's share of the rows' minimum terms: its two sub-blocks
      const float2 xs = lds64f(xsum + 256u + (uint32_t)t * 8u);
      const float mt0 = (float)(v0 & 255u) * xs.x + (float)((v0 >> 16) & 255u) * xs.y;
      const float mt1 = (float)(v1 & 255u) * xs.x + (float)((v1 >> 16) & 255u) * xs.y;
      acc[0] += d0 * (c[0] + c[1]) - n0 * mt0;
      acc[2] += d1 * (c[2] + c[3]) - n1 * mt1;
    }
  }
};

}  // namespace ishi
