// GGUF Q6_K for the tcgen05 kernel: one weight row per thread.
//
// Block layout (210 bytes per 256 weights; reference: Sources/IshizukiKit/Core/GGMLDequant.swift
// :154-185): ql[128] low nibbles, qh[64] high bit pairs, int8 scales[16], d f16. Half n of the
// block (128 weights) takes ql[64n ..], qh[32n ..], scales[8n ..]; with l in 0..31 its four runs of
// 32 weights are
//   run 0: ql[l] & 15      | (qh[l] >> 0 & 3) << 4      run 1: ql[32 + l] & 15 | (qh[l] >> 2 & 3) << 4
//   run 2: ql[l] >> 4      | (qh[l] >> 4 & 3) << 4      run 3: ql[32 + l] >> 4 | (qh[l] >> 6 & 3) << 4
// and w = (d * scale[8n + 2 run + l / 16]) * (q - 32).
//
// A step is one half n: eight groups of sixteen weights, each with its own int8 scale, each one
// K = 16 MMA into its own accumulator. scale * (q - 32) can reach 4096 and is not an exact fp16
// number, so the scale stays in fp32 and A holds q - 32: the six bits are assembled in 16-bit
// lanes on top of the fp16 bit pattern of 1024 and one half2 subtraction of 1056 makes them
// exact signed values. In the tiled copy the block is split into its four fields so that each is
// naturally aligned. Slot order inside every four k: 0, 2, 1, 3 (as for Q4_K).
#pragma once
#include "ishi_rowstream.cuh"

namespace ishi {

struct RowQ6K {
  static constexpr bool kHasMin = false;
  static constexpr int kTableBytes = 0;
  static __device__ __forceinline__ void build_table(uint8_t *, int, int) {}

  struct RowState {
    float d;
    float cs[8], ps[8];
  };
  static __device__ __forceinline__ void init_state(RowState &, uint32_t) {}

  static __device__ __forceinline__ void begin_unit(RowState &rs, const RowArgs &a, uint32_t ra, int r) {
    rs.d = half_bits_to_float(lds16(ra + a.sec_off[3] + (uint32_t)r * 2u));
  }

  static __device__ __forceinline__ uint32_t centred(uint32_t lanes) {
    // lanes hold 1024 + q as fp16 bit patterns; subtract 1056 = 1024 + 32
    const __half2 v = __hsub2(*reinterpret_cast<const __half2 *>(&lanes), __float2half2_rn(1056.f));
    return *reinterpret_cast<const uint32_t *>(&v);
  }

  static __device__ __forceinline__ void decode_step(RowState &rs, const RowArgs &a, uint32_t ra, int r, int hh,
                                                     uint32_t acol) {
    const uint32_t la = ra + a.sec_off[0] + (uint32_t)r * 128u + (uint32_t)hh * 64u;
    const uint32_t ha = ra + a.sec_off[1] + (uint32_t)r * 64u + (uint32_t)hh * 32u;
    uint32_t W[16], Hq[8];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 q = lds128(la + 16 * c);
      W[4 * c] = q.x; W[4 * c + 1] = q.y; W[4 * c + 2] = q.z; W[4 * c + 3] = q.w;
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint4 q = lds128(ha + 16 * c);
      Hq[4 * c] = q.x; Hq[4 * c + 1] = q.y; Hq[4 * c + 2] = q.z; Hq[4 * c + 3] = q.w;
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      uint32_t o[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t w = (t & 1) ? W[8 + i] : W[i];
        const uint32_t wn = (t & 2) ? (w >> 4) : w;
        const uint32_t hb = Hq[i] >> (2 * t);
        // weights (l0, l2) and (l1, l3) of the word
        o[2 * i] = centred(and_or(wn, 0x000f000fu, ((hb << 4) & 0x00300030u) | 0x64006400u));
        o[2 * i + 1] = centred(and_or(wn >> 8, 0x000f000fu, ((hb >> 4) & 0x00300030u) | 0x64006400u));
      }
      tmem_st16(acol + 16u * t, o);
    }
    const uint2 sc = lds64(ra + a.sec_off[2] + (uint32_t)r * 16u + (uint32_t)hh * 8u);
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      const uint32_t word = g < 4 ? sc.x : sc.y;
      const int v = (int)(signed char)((word >> (8 * (g & 3))) & 0xffu);
      rs.cs[g] = rs.d * (float)v;
    }
  }

  static __device__ __forceinline__ void store_min(const RowState &, int, uint32_t) {}
  static __device__ __forceinline__ void advance(RowState &rs, int, uint32_t) {
#pragma unroll
    for (int g = 0; g < 8; ++g) rs.ps[g] = rs.cs[g];
  }

  template <int MC>
  static __device__ __forceinline__ void consume_step(const RowState &rs, const RowArgs &, float (&acc)[MC],
                                                      uint32_t tlane) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float dg[4][MC];
#pragma unroll
      for (int g = 0; g < 4; ++g) tmem_ldn<MC>(tlane + kColD + 16u * (4 * half + g), dg[g]);
      tc_wait_ld();
#pragma unroll
      for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int m = 0; m < MC; ++m) acc[m] = fmaf(rs.ps[4 * half + g], dg[g][m], acc[m]);
    }
  }

  static __device__ __forceinline__ void issue_step(const RowArgs &, uint32_t tmem, uint32_t acol, uint64_t xdesc,
                                                    uint64_t, int) {
#pragma unroll
    for (int g = 0; g < 8; ++g) umma_f16(tmem + kColD + 16u * g, acol + 8u * g, xdesc + (uint64_t)(g * 16), kIdescF16, 0u);
  }

  static constexpr int kXRegs = 16;
  struct XRegs {
    uint4 v[kXRegs];
  };
  static __device__ __forceinline__ void load_x(const RowArgs &a, int u0, int nu, int lane, XRegs &xr) {
    const int m = lane & 7, gq = lane >> 3;
    const bool live = m < a.M;
    const __half *xp = a.x + (long long)(live ? m : 0) * a.K + (long long)u0 * 256 + 8 * gq;
#pragma unroll
    for (int sb = 0; sb < kXRegs; ++sb) {
      xr.v[sb] = make_uint4(0u, 0u, 0u, 0u);
      if (live && sb < 8 * nu) xr.v[sb] = __ldg(reinterpret_cast<const uint4 *>(xp + 32 * sb));
    }
  }
  static __device__ __forceinline__ void store_x(const RowArgs &a, uint32_t stage, int nu, int lane,
                                                 const XRegs &xr) {
    const int m = lane & 7, gq = lane >> 3;
#pragma unroll
    for (int sb = 0; sb < kXRegs; ++sb) {
      if (sb < 8 * nu) {
        const uint4 &v = xr.v[sb];
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(stage + a.x_off + (uint32_t)(sb * 4 + gq) * 128u +
                                                                    (uint32_t)m * 16u),
                     "r"(prmt(v.x, v.y, 0x5410u)), "r"(prmt(v.x, v.y, 0x7632u)), "r"(prmt(v.z, v.w, 0x5410u)),
                     "r"(prmt(v.z, v.w, 0x7632u))
                     : "memory");
      }
    }
  }
};

}  // namespace ishi
