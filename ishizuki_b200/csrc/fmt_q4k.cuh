// GGUF Q4_K inside the streaming kernel.
//
// Block layout (144 bytes per 256 weights; reference: Sources/IshizukiKit/Core/GGMLDequant.swift
// :187-220 and the kernel body at Sources/IshizukiKit/Core/GGMLKernels.swift:586-603):
//   d f16 @0, dmin f16 @2, twelve bytes of 6-bit (scale, min) pairs @4, 128 nibble bytes @16.
//   Byte l of 32-byte chunk j holds weight 64j + l (low nibble, sub-block 2j) and weight
//   64j + 32 + l (high nibble, sub-block 2j + 1);  w = d * sc * q - dmin * m.
//
// The product is factored per sub-block, as the reference's matvec does
// (GGMLKernels.swift:432-440):  y += d * sum_sb sc_sb * (sum_k q_k x_k) - dmin * sum_sb m_sb * (sum_k x_k).
// The codes reach the tensor core as exact fp16 numbers without a conversion instruction: a
// nibble masked in place is the bit pattern of the fp16 value q * 2^-24 (low nibble) or
// q * 2^-20 (high nibble), and the power of two is folded into the fp32 sub-block scale.
//
// Fragment mapping (m16n8k16; thread g = lane / 4, t = lane % 4 holds weight rows g and g + 8):
// in chunk j thread t reads bytes 8t .. 8t+7, one word per k-step s in {0, 1}; within the word
// the low nibbles of bytes (0, 2) and (1, 3) form the two A registers of a row, so a k-step
// covers k = 64j + 32h + 8t + 4s + {0, 2, 1, 3} and the activations are gathered in the same order.
#pragma once
#include "ishi_stream.cuh"

namespace ishi {

struct FmtQ4K {
  static constexpr int kUnitBytes = 144;
  static constexpr int kRowSkew = 32;  // row slots 32 mod 128 bytes apart: 64-bit reads of four rows never share a bank

  template <int MT, int UW>
  struct XFrag {
    uint32_t b[UW][MT][16][2];  // activation fragments per k-step (step = 4j + 2h + s)
    uint32_t xs[UW][MT][2];     // per-sub-block activation sums, split in fp16 hi / lo parts
  };

  template <int MT, int UW>
  static __device__ __forceinline__ void load_x(XFrag<MT, UW> &xf, const StreamArgs &a, int ub0,
                                                int uc, int warp, int W, int g, int t, int lane) {
    (void)lane;
#pragma unroll
    for (int q = 0; q < UW; ++q) {
      const int u = warp + q * W;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int m = mt * 8 + g;
        const bool live = u < uc && m < a.M;
        const __half *xr = a.x + (long long)(live ? m : 0) * a.K + (long long)(ub0 + (live ? u : 0)) * 256;
        float ps[8];
#pragma unroll
        for (int sb = 0; sb < 8; ++sb) ps[sb] = 0.f;
#pragma unroll
        for (int st = 0; st < 16; ++st) {
          const int j = st >> 2, h = (st >> 1) & 1, s = st & 1;
          uint2 v = make_uint2(0u, 0u);
          if (live) v = __ldg(reinterpret_cast<const uint2 *>(xr + 64 * j + 32 * h + 8 * t + 4 * s));
          xf.b[q][mt][st][0] = prmt(v.x, v.y, 0x5410);  // (x[+0], x[+2])
          xf.b[q][mt][st][1] = prmt(v.x, v.y, 0x7632);  // (x[+1], x[+3])
          const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&v.x));
          const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
          ps[2 * j + h] += (f0.x + f0.y) + (f1.x + f1.y);
        }
        // sum over the four threads that share an activation row, then keep sub-blocks 2t, 2t+1
        float keep0 = 0.f, keep1 = 0.f;
#pragma unroll
        for (int sb = 0; sb < 8; ++sb) {
          float v = ps[sb];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          if ((sb >> 1) == t) {
            if (sb & 1) keep1 = v; else keep0 = v;
          }
        }
        const __half h0 = __float2half_rn(keep0), h1 = __float2half_rn(keep1);
        const __half l0 = __float2half_rn(keep0 - __half2float(h0));
        const __half l1 = __float2half_rn(keep1 - __half2float(h1));
        xf.xs[q][mt][0] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
        xf.xs[q][mt][1] = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16);
      }
    }
  }

  // The twelve scale bytes of one block as four words of packed bytes: sc[0..3], sc[4..7],
  // m[0..3], m[4..7] (ggml's get_scale_min_k4, done on words).
  static __device__ __forceinline__ void unpack_scales(uint32_t u0, uint32_t u1, uint32_t u2,
                                                       uint32_t (&sc)[2], uint32_t (&mn)[2]) {
    sc[0] = u0 & 0x3f3f3f3fu;
    mn[0] = u1 & 0x3f3f3f3fu;
    sc[1] = and_or(u2, 0x0f0f0f0fu, (u0 >> 2) & 0x30303030u);
    mn[1] = and_or(u2 >> 4, 0x0f0f0f0fu, (u1 >> 2) & 0x30303030u);
  }

  // float(byte i of packed) * 2^e, exactly, through the exponent-bias trick.
  template <int E>
  static __device__ __forceinline__ float byte_scaled(uint32_t packed, int i) {
    constexpr uint32_t magic = (uint32_t)(127 + 23 + E) << 23;
    const uint32_t bits = prmt(packed, magic, 0x7650u | (uint32_t)i);
    return __uint_as_float(bits) - __uint_as_float(magic);
  }

  template <int MT, int UW>
  static __device__ __forceinline__ void unit(float (&acc)[MT][4], const XFrag<MT, UW> &xf, int q,
                                              const StreamArgs &a, uint32_t stage, long long row0,
                                              int first_unit, int ulocal, int g, int t) {
    (void)row0;
    (void)first_unit;
    // Q4_K rows are multiples of 16 bytes, so segments sit at the start of their row slots.
    const uint32_t r0 = stage + (uint32_t)g * a.row_stride + (uint32_t)ulocal * kUnitBytes;
    const uint32_t r1 = r0 + 8u * a.row_stride;
    const uint4 h0 = lds128(r0), h1 = lds128(r1);
    uint32_t sc0[2], mn0[2], sc1[2], mn1[2];
    unpack_scales(h0.y, h0.z, h0.w, sc0, mn0);
    unpack_scales(h1.y, h1.z, h1.w, sc1, mn1);

    float accu[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) accu[mt][0] = accu[mt][1] = accu[mt][2] = accu[mt][3] = 0.f;

#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint2 w0 = lds64(r0 + 16 + 32 * j + 8 * t);
      const uint2 w1 = lds64(r1 + 16 + 32 * j + 8 * t);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t mask = h ? 0x00f000f0u : 0x000f000fu;
        float part[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) part[mt][0] = part[mt][1] = part[mt][2] = part[mt][3] = 0.f;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const uint32_t x0 = s ? w0.y : w0.x;
          const uint32_t x1 = s ? w1.y : w1.x;
          const uint32_t a0 = x0 & mask, a1 = x1 & mask;
          const uint32_t a2 = (x0 >> 8) & mask, a3 = (x1 >> 8) & mask;
          const int st = 4 * j + 2 * h + s;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            mma16816(part[mt], a0, a1, a2, a3, xf.b[q][mt][st][0], xf.b[q][mt][st][1]);
        }
        const int sb = 2 * j + h;
        // sc * 2^24 for low nibbles (codes were q * 2^-24), sc * 2^20 for high ones (q * 2^-20)
        const float s0 = h ? byte_scaled<20>(sc0[sb >> 2], sb & 3) : byte_scaled<24>(sc0[sb >> 2], sb & 3);
        const float s1 = h ? byte_scaled<20>(sc1[sb >> 2], sb & 3) : byte_scaled<24>(sc1[sb >> 2], sb & 3);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          accu[mt][0] = fmaf(s0, part[mt][0], accu[mt][0]);
          accu[mt][1] = fmaf(s0, part[mt][1], accu[mt][1]);
          accu[mt][2] = fmaf(s1, part[mt][2], accu[mt][2]);
          accu[mt][3] = fmaf(s1, part[mt][3], accu[mt][3]);
        }
      }
    }

    // minimum term: one MMA whose k index runs over sub-blocks (hi parts in k 0..7, lo in 8..15)
    const uint32_t m0w = t < 2 ? mn0[0] : mn0[1];
    const uint32_t m1w = t < 2 ? mn1[0] : mn1[1];
    const uint32_t msel = (t & 1) ? 0x4342u : 0x4140u;  // (byte 2t', zero, byte 2t'+1, zero), t' = t % 2
    const uint32_t ma = prmt(m0w, 0u, msel);  // (m[2t], m[2t+1]) of row g as fp16 m * 2^-24
    const uint32_t mb = prmt(m1w, 0u, msel);  // row g + 8
    const float d0 = half_bits_to_float(h0.x & 0xffffu);
    const float d1 = half_bits_to_float(h1.x & 0xffffu);
    const float n0 = half_bits_to_float(h0.x >> 16) * 16777216.f;
    const float n1 = half_bits_to_float(h1.x >> 16) * 16777216.f;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float cm[4] = {0.f, 0.f, 0.f, 0.f};
      mma16816(cm, ma, mb, ma, mb, xf.xs[q][mt][0], xf.xs[q][mt][1]);
      acc[mt][0] += d0 * accu[mt][0] - n0 * cm[0];
      acc[mt][1] += d0 * accu[mt][1] - n0 * cm[1];
      acc[mt][2] += d1 * accu[mt][2] - n1 * cm[2];
      acc[mt][3] += d1 * accu[mt][3] - n1 * cm[3];
    }
  }
};

}  // namespace ishi
