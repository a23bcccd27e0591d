// GGUF IQ2_XS for the tcgen05 kernel: one weight row per thread.
//
// Block layout (74 bytes per 256 weights; reference: Sources/IshizukiKit/Core/GGMLDequant.swift
// :264-285): d f16 @0, 32 x u16 @2 (bits 0-8 index into the 512-entry grid of eight magnitudes
// out of {8, 25, 43}, bits 9-15 seven sign bits, the eighth being their parity), eight scale bytes
// @66 (low nibble: first sixteen weights of a 32-group, high nibble: the second sixteen);
// w = d * (0.5 + s) * 0.25 * grid * sign = (d / 8) * [(2s + 1) * grid * sign].
//
// The bracket is an integer of magnitude at most 31 * 43 = 1333 < 2048, so it is an exact fp16
// number and, written as raw bits, the fp16 value n * 2^-24: the sub-scale is folded into the A
// operand with one integer multiply per register pair and a whole block needs a single fp32
// scale, d / 8 * 2^24. One accumulation group per step; no minimum term.
//
// In the tiled copy a block is split into three sections (index words, scale bytes, d) so that
// each is naturally aligned. The grid sits in shared memory as two 4-byte planes per entry.
// A 16-bit lane pair (a, b) of one grid word holds magnitudes (g0, g2) / (g1, g3) after a mask,
// so inside every four k the activations are stored in the order 0, 2, 1, 3 as for Q4_K.
#pragma once
#include "dequant.cuh"
#include "ishi_rowstream.cuh"

namespace ishi {

struct RowIQ2XS {
  static constexpr bool kHasMin = false;
  static constexpr int kTableBytes = 4096;

  struct RowState {
    uint32_t tbl;       // shared-memory address of the expanded grid
    float cs, ps;       // d / 8 * 2^24 of the unit being decoded / still in tensor memory
    uint32_t sc[2];     // the unit's eight scale bytes
  };

  // 512 entries x 8 bytes: the eight magnitudes of an entry, byte j = weight j
  static __device__ __forceinline__ void build_table(uint8_t *tbl, int tid, int nthreads) {
    for (int e = tid; e < 512; e += nthreads) {
      const uint32_t codes = c_iq2xs_codes[e];
      uint32_t w[2] = {0u, 0u};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t c = (codes >> (2 * j)) & 3u;
        const uint32_t v = c == 0 ? ISHI_IQ2XS_VALUE0 : (c == 1 ? ISHI_IQ2XS_VALUE1 : ISHI_IQ2XS_VALUE2);
        w[j >> 2] |= v << (8 * (j & 3));
      }
      reinterpret_cast<uint2 *>(tbl)[e] = make_uint2(w[0], w[1]);
    }
  }

  static __device__ __forceinline__ void init_state(RowState &rs, uint32_t tbl) { rs.tbl = tbl; }

  static __device__ __forceinline__ void begin_unit(RowState &rs, const RowArgs &a, uint32_t ra, int r) {
    const uint2 s = lds64(ra + a.sec_off[1] + (uint32_t)r * 8u);
    rs.sc[0] = s.x;
    rs.sc[1] = s.y;
    rs.cs = half_bits_to_float(lds16(ra + a.sec_off[2] + (uint32_t)r * 2u)) * (16777216.f / 8.f);
  }

  // eight weights of one index word -> four A registers
  static __device__ __forceinline__ void decode8(const RowState &rs, uint32_t q, uint32_t mult, uint32_t (&o)[4]) {
    const uint2 e = lds64(rs.tbl + (q & 511u) * 8u);
    const uint32_t s7 = q >> 9;
    const uint32_t s8 = s7 | ((__popc(s7) & 1u) << 7);
    const uint32_t p0 = (e.x & 0x00ff00ffu) * mult;         // (g0, g2) * (2s + 1)
    const uint32_t p1 = ((e.x >> 8) & 0x00ff00ffu) * mult;  // (g1, g3)
    const uint32_t p2 = (e.y & 0x00ff00ffu) * mult;         // (g4, g6)
    const uint32_t p3 = ((e.y >> 8) & 0x00ff00ffu) * mult;  // (g5, g7)
    o[0] = and_xor(s8 * ((1u << 15) | (1u << 29)), 0x80008000u, p0);  // signs 0 and 2
    o[1] = and_xor(s8 * ((1u << 14) | (1u << 28)), 0x80008000u, p1);  // 1 and 3
    o[2] = and_xor(s8 * ((1u << 11) | (1u << 25)), 0x80008000u, p2);  // 4 and 6
    o[3] = and_xor(s8 * ((1u << 10) | (1u << 24)), 0x80008000u, p3);  // 5 and 7
  }

  static __device__ __forceinline__ void decode_step(RowState &rs, const RowArgs &a, uint32_t ra, int r, int hh,
                                                     uint32_t acol) {
    const uint32_t qa = ra + a.sec_off[0] + (uint32_t)r * 64u + (uint32_t)hh * 32u;
    const uint32_t scw = rs.sc[hh];  // four scale bytes: 32-groups 4hh .. 4hh+3
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint4 q = lds128(qa + 16 * c);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 2; ++i) {  // one 32-group = two words = four index entries = sixteen columns
        const uint32_t sb = (scw >> (8 * (2 * c + i))) & 0xffu;
        const uint32_t mlo = 2u * (sb & 0xfu) + 1u, mhi = 2u * (sb >> 4) + 1u;
        uint32_t o[16], t[4];
        decode8(rs, w[2 * i] & 0xffffu, mlo, t);
        o[0] = t[0]; o[1] = t[1]; o[2] = t[2]; o[3] = t[3];
        decode8(rs, w[2 * i] >> 16, mlo, t);
        o[4] = t[0]; o[5] = t[1]; o[6] = t[2]; o[7] = t[3];
        decode8(rs, w[2 * i + 1] & 0xffffu, mhi, t);
        o[8] = t[0]; o[9] = t[1]; o[10] = t[2]; o[11] = t[3];
        decode8(rs, w[2 * i + 1] >> 16, mhi, t);
        o[12] = t[0]; o[13] = t[1]; o[14] = t[2]; o[15] = t[3];
        tmem_st16(acol + 16u * (2 * c + i), o);
      }
    }
  }

  static __device__ __forceinline__ void store_min(const RowState &, int, uint32_t) {}
  static __device__ __forceinline__ void advance(RowState &rs, int, uint32_t) { rs.ps = rs.cs; }

  template <int MC>
  static __device__ __forceinline__ void consume_step(const RowState &rs, const RowArgs &, float (&acc)[MC],
                                                      uint32_t tlane) {
    float d[MC];
    tmem_ldn<MC>(tlane + kColD, d);
    tc_wait_ld();
#pragma unroll
    for (int m = 0; m < MC; ++m) acc[m] = fmaf(rs.ps, d[m], acc[m]);
  }

  static __device__ __forceinline__ void issue_step(const RowArgs &, uint32_t tmem, uint32_t acol, uint64_t xdesc,
                                                    uint64_t, int) {
#pragma unroll
    for (int j = 0; j < 8; ++j) umma_f16(tmem + kColD, acol + 8u * j, xdesc + (uint64_t)(j * 16), kIdescF16, j > 0 ? 1u : 0u);
  }

  // activation warp: same slot order as Q4_K (0, 2, 1, 3 inside every four k), no group sums
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
