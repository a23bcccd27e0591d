// GGUF Q4_K for the warp-level kernel (mma.sync fragments, or CUDA-core FMA for one row).
//
// Block layout (144 bytes per 256 weights; reference: Sources/IshizukiKit/Core/GGMLDequant.swift
// :187-220 and the kernel body at Sources/IshizukiKit/Core/GGMLKernels.swift:586-603):
//   d f16 @0, dmin f16 @2, twelve bytes of 6-bit (scale, min) pairs @4, 128 nibble bytes @16.
//   Byte l of 32-byte chunk j holds weight 64j + l (low nibble, sub-block 2j) and weight
//   64j + 32 + l (high nibble, sub-block 2j + 1);  w = d * sc * q - dmin * m.
//
// The product is factored per sub-block as the reference's matvec does
// (GGMLKernels.swift:432-440): y += d * sum_sb sc_sb * (sum_k q_k x_k) - dmin * sum_sb m_sb * (sum_k x_k).
// A nibble masked in place is the bit pattern of the fp16 number q * 2^-24 (low) or q * 2^-20
// (high), so a fragment register costs one AND (plus one shift per word); the power of two goes
// into the fp32 sub-block scale.
//
// Fragment mapping (m16n8k16; lane g = lane / 4, t = lane % 4 holds weight rows g and g + 8): in
// chunk j lane t owns bytes 8t .. 8t+7 of both rows, one word per k-step s in {0, 1}; within a word
// the low nibbles of bytes (0, 2) and (1, 3) form the two A registers of a row, so k-step
// (j, h, s) covers k = 64j + 32h + 8t + 4s + {0, 2, 1, 3} and x is staged in that order.
// Tile (16 rows x 256 k, 2304 bytes): piece j = [lane][row g: 8 bytes, row g + 8: 8 bytes] for
// j = 0..3, then the sixteen 16-byte block headers.
#pragma once
#include "ishi_fragstream.cuh"

namespace ishi {

struct FragQ4K {
  static constexpr int kTileBytes = 16 * 144;
  static constexpr int kXBytes = 4480;  // 16 k-steps x 256 B fragments, 256 B sub-block sums (fp16 hi/lo), 32 B fp32 sums of row 0

  static __device__ __forceinline__ uint16_t tile_halfword(const FragSrc &s, long long p, int u, int hw) {
    int row_in_panel, off;
    if (hw < 1024) {
      const int c = hw >> 8, lane = (hw & 255) >> 3, h = hw & 7;
      const int g = lane >> 2, t = lane & 3;
      row_in_panel = g + 8 * (h >> 2);
      off = 16 + 32 * c + 8 * t + 2 * (h & 3);
    } else {
      const int idx = hw - 1024;
      row_in_panel = idx >> 3;
      off = 2 * (idx & 7);
    }
    const long long row = p * kFragRows + row_in_panel;
    if (row >= s.N) return 0;
    long long local;
    const int seg = frag_segment(s, row, &local);
    return *reinterpret_cast<const uint16_t *>(s.w[seg] + local * s.w_row_bytes + (long long)u * 144 + off);
  }

  // Activations of the CTA's column range into fragment order. A warp task is (unit, activation
  // row): lane l loads the eight values k = 8l .. 8l+7 of the unit (both k-steps s of chunk
  // j = l / 8, half h = (l / 4) % 2, t = l % 4), so a task is one contiguous 512-byte read. The
  // fragment of k-step st = 4j + 2h + s sits at st * 256 + ((g ^ j) * 4 + t) * 8: the xor spreads
  // the four chunks of a store over the banks, and a k-step's 32 lanes still read one 256-byte run.
  // after_loads() runs once, when the first batch of loads is in flight and before their values are
  // used (the kernel issues its first weight copies there, behind the activations).
  template <class F>
  static __device__ __forceinline__ void stage_x(const FragArgs &a, uint32_t xfrag, int ub0, int uc, F &&after_loads) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int tasks = uc * 8;
    constexpr int kBatch = 8;
    const int jj = lane >> 3, hh = (lane >> 2) & 1, tt = lane & 3;
    const __half *xl = a.x + (long long)ub0 * 256 + lane * 8;
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
        const uint32_t dst = base + (uint32_t)(4 * jj + 2 * hh) * 256u + (uint32_t)(((g ^ jj) * 4 + tt) * 8);
        sts64(dst, prmt(v[e].x, v[e].y, 0x5410u), prmt(v[e].x, v[e].y, 0x7632u));
        sts64(dst + 256u, prmt(v[e].z, v[e].w, 0x5410u), prmt(v[e].z, v[e].w, 0x7632u));
        // sums of x over the sub-block (four lanes), for the minimum term
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].y));
        const float2 f2 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].z));
        const float2 f3 = __half22float2(*reinterpret_cast<const __half2 *>(&v[e].w));
        float s = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        const float o = __shfl_xor_sync(0xffffffffu, s, 4);
        if ((lane & 7) == 0) {
          // sub-blocks 2t' and 2t'+1 (t' = lane / 8) of activation row g, as fp16 hi + lo
          const __half h0 = __float2half_rn(s), h1 = __float2half_rn(o);
          const __half l0 = __float2half_rn(s - __half2float(h0)), l1 = __float2half_rn(o - __half2float(h1));
          sts64(base + 4096u + (uint32_t)(g * 4 + jj) * 8u,
                (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16),
                (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16));
        }
        if (g == 0 && tt == 0)  // fp32 sums of activation row 0 (the single-row kernel's minimum term)
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(base + 4352u + (uint32_t)(lane >> 2) * 4u), "f"(s) : "memory");
      }
    }
  }

  // The twelve scale bytes of one block as packed bytes: sc[0..3], sc[4..7], m[0..3], m[4..7]
  // (ggml's get_scale_min_k4, done on words).
  static __device__ __forceinline__ void unpack_scales(uint32_t u0, uint32_t u1, uint32_t u2, uint32_t (&sc)[2],
                                                       uint32_t (&mn)[2]) {
    sc[0] = u0 & 0x3f3f3f3fu;
    mn[0] = u1 & 0x3f3f3f3fu;
    sc[1] = and_or(u2, 0x0f0f0f0fu, (u0 >> 2) & 0x30303030u);
    mn[1] = and_or(u2 >> 4, 0x0f0f0f0fu, (u1 >> 2) & 0x30303030u);
  }

  // float(byte i of packed) * 2^E, exactly, through the exponent-bias trick
  template <int E>
  static __device__ __forceinline__ float byte_scaled(uint32_t packed, int i) {
    constexpr uint32_t magic = (uint32_t)(127 + 23 + E) << 23;
    return __uint_as_float(prmt(packed, magic, 0x7650u | (uint32_t)i)) - __uint_as_float(magic);
  }

  static __device__ __forceinline__ float half_lo(uint32_t pair) { return __half2float(__ushort_as_half((unsigned short)(pair & 0xffffu))); }
  static __device__ __forceinline__ float half_hi(uint32_t pair) { return __half2float(__ushort_as_half((unsigned short)(pair >> 16))); }

  // One tile against the activations of its unit. acc: the warp's C fragment (MODE 0) or this
  // lane's partial dot products of rows g (acc[0]) and g + 8 (acc[2]) (MODE 1).
  template <int MODE>
  static __device__ __forceinline__ void unit(float (&acc)[4], const FragArgs &a, uint32_t tile, uint32_t xu, int g,
                                              int t, int lane) {
    (void)a;
    const uint4 h0 = lds128(tile + 2048u + (uint32_t)g * 16u), h1 = lds128(tile + 2048u + (uint32_t)(g + 8) * 16u);
    uint32_t sc0[2], mn0[2], sc1[2], mn1[2];
    unpack_scales(h0.y, h0.z, h0.w, sc0, mn0);
    unpack_scales(h1.y, h1.z, h1.w, sc1, mn1);
    float accu[4] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t xl = xu + (uint32_t)(MODE == 0 ? lane : t) * 8u;  // single row: the fragments of activation row 0
    // (xu is 128-byte aligned, so the staging swizzle is an xor on the address)

#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 w = lds128(tile + (uint32_t)j * 512u + (uint32_t)lane * 16u);  // row g: w.x, w.y; row g + 8: w.z, w.w
      const uint32_t xj = xl ^ (uint32_t)(j << 5);  // the chunk's staging swizzle; k-steps follow at 256-byte steps
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t mask = h ? 0x00f000f0u : 0x000f000fu;
        float part[4];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const uint32_t x0 = s ? w.y : w.x, x1 = s ? w.w : w.z;
          const uint32_t a0 = x0 & mask, a1 = x1 & mask, a2 = (x0 >> 8) & mask, a3 = (x1 >> 8) & mask;
          const uint2 b = lds64(xj + (uint32_t)(4 * j + 2 * h + s) * 256u);
          if (MODE == 0) {
            if (s == 0) mma16816_first(part, a0, a1, a2, a3, b.x, b.y);
            else mma16816(part, a0, a1, a2, a3, b.x, b.y);
          } else {
            if (s == 0) part[0] = part[1] = part[2] = part[3] = 0.f;
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
        const int sb = 2 * j + h;
        const float s0 = h ? byte_scaled<20>(sc0[sb >> 2], sb & 3) : byte_scaled<24>(sc0[sb >> 2], sb & 3);
        const float s1 = h ? byte_scaled<20>(sc1[sb >> 2], sb & 3) : byte_scaled<24>(sc1[sb >> 2], sb & 3);
        accu[0] = fmaf(s0, part[0], accu[0]);
        accu[1] = fmaf(s0, part[1], accu[1]);
        accu[2] = fmaf(s1, part[2], accu[2]);
        accu[3] = fmaf(s1, part[3], accu[3]);
      }
    }

    const float d0 = half_bits_to_float(h0.x & 0xffffu), d1 = half_bits_to_float(h1.x & 0xffffu);
    if (MODE == 0) {
      // minimum term: one MMA whose k index runs over sub-blocks (hi parts in k 0..7, lo in 8..15)
      const uint32_t m0w = t < 2 ? mn0[0] : mn0[1], m1w = t < 2 ? mn1[0] : mn1[1];
      const uint32_t msel = (t & 1) ? 0x4342u : 0x4140u;  // (byte 2t', zero, byte 2t'+1, zero), t' = t % 2
      const uint32_t ma = prmt(m0w, 0u, msel), mb = prmt(m1w, 0u, msel);  // (m[2t], m[2t+1]) as fp16 m * 2^-24
      const uint2 xs = lds64(xu + 4096u + (uint32_t)lane * 8u);
      float cm[4];
      mma16816_first(cm, ma, mb, ma, mb, xs.x, xs.y);
      const float n0 = half_bits_to_float(h0.x >> 16) * 16777216.f, n1 = half_bits_to_float(h1.x >> 16) * 16777216.f;
      acc[0] += d0 * accu[0] - n0 * cm[0];
      acc[1] += d0 * accu[1] - n0 * cm[1];
      acc[2] += d1 * accu[2] - n1 * cm[2];
      acc[3] += d1 * accu[3] - n1 * cm[3];
    } else {
      // the row's minimum term enters once: lane t = 0 of the row adds it
      float mt0 = 0.f, mt1 = 0.f;
      if (t == 0) {
        const float4 xa = lds128f(xu + 4352u), xb = lds128f(xu + 4368u);
        const float xs[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int sb = 0; sb < 8; ++sb) {
          mt0 = fmaf(byte_scaled<0>(mn0[sb >> 2], sb & 3), xs[sb], mt0);
          mt1 = fmaf(byte_scaled<0>(mn1[sb >> 2], sb & 3), xs[sb], mt1);
        }
      }
      acc[0] += d0 * accu[0] - half_bits_to_float(h0.x >> 16) * mt0;
      acc[2] += d1 * accu[2] - half_bits_to_float(h1.x >> 16) * mt1;
    }
  }
};

}  // namespace ishi
