// MLX affine group-quantized packs (2, 4 or 8 bits) for the tcgen05 kernel.
//
// Layout (reference: Sources/IshizukiKit/Core/VerifyMatmul.swift:282-287 and
// Sources/IshizukiKit/Quantize/WeightedAffineQuantizer.swift:142-161): row n is K*bits/32
// little-endian uint32 words, code i at bit i*bits; w = float(code) * scale + bias with one
// (scale, bias) pair per group of group_size inputs, stored as fp16, bf16 or fp32.
//
// The product is factored per group as the reference's codes kernel does
// (VerifyMatmul.swift:123-128): y += s_g * sum_k code_k x_k + b_g * sum_k x_k. The first sum is
// the tensor core's: codes masked in place are fp16 bit patterns of code * 2^-24 times the power
// of two of their bit position (a 4-bit code in bits 4..7 reads as 16 * code, and so on); that
// extra power of two is taken out on the activation side, where x is stored divided by it
// (exact unless |x| is below 2^-8 or so, where it costs at most half a unit in the last place of
// an fp16 subnormal). The second sum is an fp32 group sum of x the activation warp leaves in
// shared memory, applied with the bias by each row's thread, so any scale dtype works.
//
// Slot order inside one word (the order x is stored in):
//   4 bits: k0 k4 | k1 k5 (x/16) | k2 k6 | k3 k7 (x/16)
//   2 bits: k0 k8 | k1 k9 (x/4) | k2 k10 (x/16) | k3 k11 (x/64) | k4 k12 | k5 k13 (x/4) | ...
//   8 bits: k0 k2 | k1 k3
#pragma once
#include <cuda_bf16.h>

#include "ishi_rowstream.cuh"

namespace ishi {

template <int BITS>
struct RowAffine {
  static_assert(BITS == 2 || BITS == 4 || BITS == 8, "affine widths with a whole number of codes per word");
  static constexpr bool kHasMin = false;
  static constexpr int kTableBytes = 0;
  static __device__ __forceinline__ void build_table(uint8_t *, int, int) {}
  static constexpr int kCodeBytes = 32 * BITS;   // per row per unit
  static constexpr int kStepBytes = 16 * BITS;   // per row per 128-k step

  struct RowState {
    float cs[4], cb[4];  // scale * 2^24 and bias of the groups of the step being decoded
    float ps[4], pb[4];  // ... of the step whose accumulators are still in tensor memory
    uint32_t pxs;        // shared-memory address of that step's group sums of x
  };

  static __device__ __forceinline__ float load_param(uint32_t addr, int dtype) {
    if (dtype == 2) return __uint_as_float(lds32(addr));
    const uint32_t h = lds16(addr);
    return dtype == 0 ? half_bits_to_float(h) : bf16_bits_to_float(h);
  }

  static __device__ __forceinline__ void init_state(RowState &, uint32_t) {}
  static __device__ __forceinline__ void begin_unit(RowState &, const RowArgs &, uint32_t, int) {}

  static __device__ __forceinline__ void decode_step(RowState &rs, const RowArgs &a, uint32_t ra, int r, int hh,
                                                     uint32_t acol) {
    const uint32_t ca = ra + a.sec_off[0] + (uint32_t)r * kCodeBytes + (uint32_t)hh * kStepBytes;
    if (BITS == 4) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {  // four words -> sixteen columns
        const uint4 q = lds128(ca + 16 * c);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint32_t o[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t s8 = w[i] >> 8;
          o[4 * i + 0] = w[i] & 0x000f000fu;
          o[4 * i + 1] = w[i] & 0x00f000f0u;
          o[4 * i + 2] = s8 & 0x000f000fu;
          o[4 * i + 3] = s8 & 0x00f000f0u;
        }
        tmem_st16(acol + 16u * c, o);
      }
    } else if (BITS == 2) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint4 q = lds128(ca + 16 * c);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t o[16];
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const uint32_t v = w[2 * half + i], s8 = v >> 8;
            o[8 * i + 0] = v & 0x00030003u;
            o[8 * i + 1] = v & 0x000c000cu;
            o[8 * i + 2] = v & 0x00300030u;
            o[8 * i + 3] = v & 0x00c000c0u;
            o[8 * i + 4] = s8 & 0x00030003u;
            o[8 * i + 5] = s8 & 0x000c000cu;
            o[8 * i + 6] = s8 & 0x00300030u;
            o[8 * i + 7] = s8 & 0x00c000c0u;
          }
          tmem_st16(acol + 32u * c + 16u * half, o);
        }
      }
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 q0 = lds128(ca + 32 * c), q1 = lds128(ca + 32 * c + 16);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        uint32_t o[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          o[2 * i] = w[i] & 0x00ff00ffu;
          o[2 * i + 1] = (w[i] >> 8) & 0x00ff00ffu;
        }
        tmem_st16(acol + 16u * c, o);
      }
    }
    // the step's group parameters
    const int G = 128 / a.group_size;
    const int pb = a.scale_dtype == 2 ? 4 : 2;
    const int per_unit = 256 / a.group_size;
    const uint32_t sa = ra + a.sec_off[1] + (uint32_t)(r * per_unit + hh * G) * pb;
    const uint32_t ba = ra + a.sec_off[2] + (uint32_t)(r * per_unit + hh * G) * pb;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      rs.cs[g] = 0.f;
      rs.cb[g] = 0.f;
      if (g < G) {
        rs.cs[g] = load_param(sa + g * pb, a.scale_dtype) * 16777216.f;
        rs.cb[g] = load_param(ba + g * pb, a.scale_dtype);
      }
    }
  }

  static __device__ __forceinline__ void store_min(const RowState &, int, uint32_t) {}

  static __device__ __forceinline__ void advance(RowState &rs, int, uint32_t xs_addr) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      rs.ps[g] = rs.cs[g];
      rs.pb[g] = rs.cb[g];
    }
    rs.pxs = xs_addr;
  }

  template <int MC>
  static __device__ __forceinline__ void consume_step(const RowState &rs, const RowArgs &a, float (&acc)[MC],
                                                      uint32_t tlane) {
    const int G = 128 / a.group_size;
    float dg[4][MC];
#pragma unroll
    for (int g = 0; g < 4; ++g)
      if (g < G) tmem_ldn<MC>(tlane + kColD + 16u * g, dg[g]);
    tc_wait_ld();
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (g < G) {
        const float4 x0 = lds128f(rs.pxs + 32u * g), x1 = lds128f(rs.pxs + 32u * g + 16u);
        const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int m = 0; m < MC; ++m) acc[m] = fmaf(rs.ps[g], dg[g][m], fmaf(rs.pb[g], xs[m], acc[m]));
      }
    }
  }

  static __device__ __forceinline__ void issue_step(const RowArgs &a, uint32_t tmem, uint32_t acol, uint64_t xdesc,
                                                    uint64_t, int) {
    const int per = a.group_size / 16;  // MMAs per group; eight MMAs a step
#pragma unroll
    for (int j = 0; j < 8; ++j)
      umma_f16(tmem + kColD + 16u * (uint32_t)(j / per), acol + 8u * j, xdesc + (uint64_t)(j * 16), kIdescF16,
               (j % per) != 0 ? 1u : 0u);
  }

  // ---- activation warp ---------------------------------------------------------------------------
  // Lane (m = lane % 8, gq = lane / 8) takes row m. Per iteration the warp covers 32 k (4 and 8
  // bits: eight k a lane) or 64 k (2 bits: sixteen k a lane, one whole word); a stage of two
  // units needs 16 resp. 8 iterations.
  static constexpr int kRun = BITS == 2 ? 16 : 8;
  static constexpr int kIters = 512 / (4 * kRun);
  struct XRegs {
    uint4 v[kIters][kRun / 8];
  };

  static __device__ __forceinline__ void load_x(const RowArgs &a, int u0, int nu, int lane, XRegs &xr) {
    const int m = lane & 7, gq = lane >> 3;
    const bool live = m < a.M;
    const __half *xp = a.x + (long long)(live ? m : 0) * a.K + (long long)u0 * 256 + kRun * gq;
#pragma unroll
    for (int it = 0; it < kIters; ++it)
#pragma unroll
      for (int h = 0; h < kRun / 8; ++h) {
        xr.v[it][h] = make_uint4(0u, 0u, 0u, 0u);
        if (live && it * 4 * kRun < 256 * nu)
          xr.v[it][h] = __ldg(reinterpret_cast<const uint4 *>(xp + it * 4 * kRun + 8 * h));
      }
  }

  static __device__ __forceinline__ float sum8(const uint4 &v) {
    const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&v.x));
    const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
    const float2 f2 = __half22float2(*reinterpret_cast<const __half2 *>(&v.z));
    const float2 f3 = __half22float2(*reinterpret_cast<const __half2 *>(&v.w));
    return ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
  }
  static __device__ __forceinline__ uint32_t scaled(uint32_t pair, float f) {
    const __half2 h = __hmul2(*reinterpret_cast<const __half2 *>(&pair), __float2half2_rn(f));
    return *reinterpret_cast<const uint32_t *>(&h);
  }
  static __device__ __forceinline__ void sts128u(uint32_t addr, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a0), "r"(a1), "r"(a2), "r"(a3) : "memory");
  }

  static __device__ __forceinline__ void store_x(const RowArgs &a, uint32_t stage, int nu, int lane,
                                                 const XRegs &xr) {
    const int m = lane & 7, gq = lane >> 3;
    const int span = 4 * kRun;  // k covered by the warp per iteration
    float run = 0.f;            // running group sum when a group spans several iterations
#pragma unroll
    for (int it = 0; it < kIters; ++it) {
      if (it * span < 256 * nu) {
        float part;
        if (BITS == 2) {
          const uint4 &A = xr.v[it][0], &B = xr.v[it][kRun / 8 - 1];
          part = sum8(A) + sum8(B);
          const uint32_t base = stage + a.x_off + (uint32_t)((it * 4 + gq) * 2) * 128u + (uint32_t)m * 16u;
          sts128u(base, prmt(A.x, B.x, 0x5410u), scaled(prmt(A.x, B.x, 0x7632u), 0.25f),
                  scaled(prmt(A.y, B.y, 0x5410u), 0.0625f), scaled(prmt(A.y, B.y, 0x7632u), 0.015625f));
          sts128u(base + 128u, prmt(A.z, B.z, 0x5410u), scaled(prmt(A.z, B.z, 0x7632u), 0.25f),
                  scaled(prmt(A.w, B.w, 0x5410u), 0.0625f), scaled(prmt(A.w, B.w, 0x7632u), 0.015625f));
        } else {
          const uint4 &A = xr.v[it][0];
          part = sum8(A);
          const uint32_t base = stage + a.x_off + (uint32_t)(it * 4 + gq) * 128u + (uint32_t)m * 16u;
          if (BITS == 4)
            sts128u(base, prmt(A.x, A.z, 0x5410u), scaled(prmt(A.x, A.z, 0x7632u), 0.0625f),
                    prmt(A.y, A.w, 0x5410u), scaled(prmt(A.y, A.w, 0x7632u), 0.0625f));
          else
            sts128u(base, prmt(A.x, A.y, 0x5410u), prmt(A.x, A.y, 0x7632u), prmt(A.z, A.w, 0x5410u),
                    prmt(A.z, A.w, 0x7632u));
        }
        // group sums of the true x: across the lanes of a row first, then across iterations
        const int gs = a.group_size;
        float s = part;
        if (gs >= 2 * kRun) s += __shfl_xor_sync(0xffffffffu, s, 8);
        if (gs >= 4 * kRun) s += __shfl_xor_sync(0xffffffffu, s, 16);
        const int k0 = it * span;  // first k of this iteration inside the stage
        if (gs >= span) {
          run = (k0 % gs == 0) ? s : run + s;
          if ((k0 + span) % gs == 0 && gq == 0) {
            const int g = k0 / gs;  // group index inside the stage (four slots per 128-k step)
            const int step = (g * gs) / 128, slot = (g * gs % 128) / gs;
            asm volatile("st.shared.f32 [%0], %1;" ::"r"(stage + a.xs_off + (uint32_t)step * 128u +
                                                           (uint32_t)slot * 32u + (uint32_t)m * 4u),
                         "f"(run)
                         : "memory");
          }
        } else {
          // several groups inside one iteration (group 32 with sixteen k a lane): lanes gq = 0, 2 hold them
          const int kk = k0 + kRun * gq;
          if ((kk % gs) == 0) {
            const int g = kk / gs;
            const int step = (g * gs) / 128, slot = (g * gs % 128) / gs;
            asm volatile("st.shared.f32 [%0], %1;" ::"r"(stage + a.xs_off + (uint32_t)step * 128u +
                                                           (uint32_t)slot * 32u + (uint32_t)m * 4u),
                         "f"(s)
                         : "memory");
          }
        }
      }
    }
  }
};

}  // namespace ishi
