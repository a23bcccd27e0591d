// GGUF Q4_K for the tcgen05 kernel: one weight row per thread.
//
// Block layout (144 bytes per 256 weights; reference: Sources/IshizukiKit/Core/GGMLDequant.swift
// :187-220): d f16 @0, dmin f16 @2, twelve bytes of 6-bit (scale, min) pairs @4, 128 nibble bytes
// @16; byte l of 32-byte chunk j is weight 64j + l (low nibble, sub-block 2j) and 64j + 32 + l
// (high nibble, sub-block 2j + 1); w = d * sc * q - dmin * m.
//
// A step is 128 k = chunks 2hh and 2hh + 1 = sub-blocks 4hh .. 4hh + 3, one accumulation group
// per sub-block. A nibble masked in place is the bit pattern of the fp16 number q * 2^-24 (low)
// or q * 2^-20 (high), so sixteen registers of a sub-block cost one AND each (plus one shift per
// word) and go to tensor memory as they are; the power of two is folded into the row's fp32
// sub-block scale d * sc. Word w of a chunk yields the pairs (4w, 4w + 2) and (4w + 1, 4w + 3), so
// inside every run of four k the activations are stored in the order 0, 2, 1, 3.
// The minimum term sum_sb m_sb * (sum_k x_k) is one more MMA per step whose K index runs over
// the step's four sub-blocks: A holds m_sb (as m * 2^-24), B the sub-block sums of x split into
// an fp16 high and low part.
#pragma once
#include "ishi_rowstream.cuh"

namespace ishi {

struct RowQ4K {
  static constexpr int kUnitBytes = 144;
  static constexpr bool kHasMin = true;
  static constexpr int kTableBytes = 0;
  static __device__ __forceinline__ void build_table(uint8_t *, int, int) {}

  struct RowState {
    float d, nmin;        // block scale, dmin * 2^24
    uint32_t sc[2], mn[2];  // packed 6-bit scales / mins of the unit
    float cs[4];          // fp32 scales of the step being decoded
    float ps[4], pmin;    // ... of the step whose accumulators are still in tensor memory
    int prev_hh;
  };

  static __device__ __forceinline__ void init_state(RowState &, uint32_t) {}

  template <int E>
  static __device__ __forceinline__ float byte_scaled(uint32_t packed, int i) {
    constexpr uint32_t magic = (uint32_t)(127 + 23 + E) << 23;
    return __uint_as_float(prmt(packed, magic, 0x7650u | (uint32_t)i)) - __uint_as_float(magic);
  }

  // ra: the unit's tile in shared memory; this thread's block is its r-th 144 bytes
  static __device__ __forceinline__ void begin_unit(RowState &rs, const RowArgs &a, uint32_t ra, int r) {
    (void)a;
    const uint4 h = lds128(ra + (uint32_t)r * kUnitBytes);
    rs.d = half_bits_to_float(h.x & 0xffffu);
    rs.nmin = half_bits_to_float(h.x >> 16) * 16777216.f;
    rs.sc[0] = h.y & 0x3f3f3f3fu;
    rs.mn[0] = h.z & 0x3f3f3f3fu;
    rs.sc[1] = and_or(h.w, 0x0f0f0f0fu, (h.y >> 2) & 0x30303030u);
    rs.mn[1] = and_or(h.w >> 4, 0x0f0f0f0fu, (h.z >> 2) & 0x30303030u);
  }

  static __device__ __forceinline__ void decode_step(RowState &rs, const RowArgs &a, uint32_t ra, int r, int hh,
                                                     uint32_t acol) {
    (void)a;
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
      const uint32_t qa = ra + (uint32_t)r * kUnitBytes + 16 + 32 * (2 * hh + jj);
      const uint4 q0 = lds128(qa), q1 = lds128(qa + 16);
      const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
      uint32_t lo[16], hi[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t s8 = w[i] >> 8;
        lo[2 * i] = w[i] & 0x000f000fu;
        lo[2 * i + 1] = s8 & 0x000f000fu;
        hi[2 * i] = w[i] & 0x00f000f0u;
        hi[2 * i + 1] = s8 & 0x00f000f0u;
      }
      tmem_st16(acol + (uint32_t)(2 * jj) * 16u, lo);
      tmem_st16(acol + (uint32_t)(2 * jj + 1) * 16u, hi);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t word = rs.sc[hh];  // sub-blocks 4hh .. 4hh+3 are the four bytes of word hh
      rs.cs[i] = ((i & 1) ? byte_scaled<20>(word, i) : byte_scaled<24>(word, i)) * rs.d;
    }
  }

  static __device__ __forceinline__ void store_min(const RowState &rs, int hh, uint32_t tlane) {
    const uint32_t m01 = prmt(rs.mn[hh], 0u, 0x4140u);  // (m0, m1) as fp16 m * 2^-24
    const uint32_t m23 = prmt(rs.mn[hh], 0u, 0x4342u);
    const uint32_t r[8] = {m01, m23, m01, m23, 0u, 0u, 0u, 0u};
    tmem_st8(tlane + kColAmin, r);
  }

  static __device__ __forceinline__ void advance(RowState &rs, int hh, uint32_t xs_addr) {
    (void)xs_addr;
#pragma unroll
    for (int i = 0; i < 4; ++i) rs.ps[i] = rs.cs[i];
    rs.pmin = rs.nmin;
    rs.prev_hh = hh;
  }

  template <int MC>
  static __device__ __forceinline__ void consume_step(const RowState &rs, const RowArgs &a, float (&acc)[MC],
                                                      uint32_t tlane) {
    (void)a;
    float dg[4][MC], dm[MC];
#pragma unroll
    for (int i = 0; i < 4; ++i) tmem_ldn<MC>(tlane + kColD + 16u * i, dg[i]);
    if (rs.prev_hh == 1) tmem_ldn<MC>(tlane + kColDmin, dm);
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int m = 0; m < MC; ++m) acc[m] = fmaf(rs.ps[i], dg[i][m], acc[m]);
    if (rs.prev_hh == 1) {
#pragma unroll
      for (int m = 0; m < MC; ++m) acc[m] = fmaf(-rs.pmin, dm[m], acc[m]);
    }
  }

  // one thread: the nine MMAs of a step
  // xdesc / mdesc: descriptors of the step's first x core matrix and of its group-sum operand; a
  // later MMA's operand is 256 bytes further, i.e. 16 more in the descriptor's address field
  static __device__ __forceinline__ void issue_step(const RowArgs &a, uint32_t tmem, uint32_t acol, uint64_t xdesc,
                                                    uint64_t mdesc, int hh) {
    (void)a;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int s = 0; s < 2; ++s)
        umma_f16(tmem + kColD + 16u * i, acol + 16u * i + 8u * s, xdesc + (uint64_t)((i * 2 + s) * 16), kIdescF16,
                 (uint32_t)s);
    umma_f16(tmem + kColDmin, tmem + kColAmin, mdesc, kIdescF16, (uint32_t)hh);
  }

  // activation warp, first half: the stage's slice of x into registers. Lane (m = lane % 8,
  // gq = lane / 8) takes eight consecutive k of row m per sub-block, so every load is issued
  // before the warp waits for the stage to be free.
  static constexpr int kXRegs = 16;  // sub-blocks per stage at most (two units)
  struct XRegs {
    uint4 v[kXRegs];
  };
  static __device__ __forceinline__ void load_x(const RowArgs &a, int u0, int nu, int lane, XRegs &xr_) {
    uint4(&v)[kXRegs] = xr_.v;
    const int m = lane & 7, gq = lane >> 3;
    const bool live = m < a.M;
    const __half *xr = a.x + (long long)(live ? m : 0) * a.K + (long long)u0 * 256 + 8 * gq;
#pragma unroll
    for (int sb = 0; sb < kXRegs; ++sb) {
      v[sb] = make_uint4(0u, 0u, 0u, 0u);
      if (live && sb < 8 * nu) v[sb] = __ldg(reinterpret_cast<const uint4 *>(xr + 32 * sb));
    }
  }

  // second half: core matrices (k order 0,2,1,3 inside every four) and the per-sub-block sums,
  // split into an fp16 high and low part, into the group-sum operand
  static __device__ __forceinline__ void store_x(const RowArgs &a, uint32_t stage, int nu, int lane,
                                                 const XRegs &xr_) {
    const uint4(&v)[kXRegs] = xr_.v;
    const int m = lane & 7, gq = lane >> 3;
#pragma unroll
    for (int sb = 0; sb < kXRegs; ++sb) {
      if (sb < 8 * nu) {
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&v[sb].x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&v[sb].y));
        const float2 f2 = __half22float2(*reinterpret_cast<const __half2 *>(&v[sb].z));
        const float2 f3 = __half22float2(*reinterpret_cast<const __half2 *>(&v[sb].w));
        float sum = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
        sum += __shfl_xor_sync(0xffffffffu, sum, 8);
        sum += __shfl_xor_sync(0xffffffffu, sum, 16);
        const uint32_t ox = prmt(v[sb].x, v[sb].y, 0x5410u), oy = prmt(v[sb].x, v[sb].y, 0x7632u);
        const uint32_t oz = prmt(v[sb].z, v[sb].w, 0x5410u), ow = prmt(v[sb].z, v[sb].w, 0x7632u);
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(stage + a.x_off + (uint32_t)(sb * 4 + gq) * 128u +
                                                                    (uint32_t)m * 16u),
                     "r"(ox), "r"(oy), "r"(oz), "r"(ow)
                     : "memory");
        if (gq == 0) {
          const __half hi = __float2half_rn(sum);
          const __half lo = __float2half_rn(sum - __half2float(hi));
          const uint32_t base =
              stage + a.bmin_off + (uint32_t)(sb >> 2) * 256u + (uint32_t)m * 16u + (uint32_t)(sb & 3) * 2u;
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(base), "h"(__half_as_ushort(hi)) : "memory");
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(base + 8u), "h"(__half_as_ushort(lo)) : "memory");
        }
      }
    }
  }
};

}  // namespace ishi
