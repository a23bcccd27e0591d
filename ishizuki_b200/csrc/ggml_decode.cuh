// Decoders of the GGML block formats, eight weights at a time: lane L of a warp decodes weights
// 8L .. 8L+7 of one 256-weight block, as the reference's Metal decoder does
// (Sources/IshizukiKit/Core/GGMLKernels.swift:391-401, bodies :568-761). These define "the decoded
// weight values": they must equal ggml's to_float (restated in
// Sources/IshizukiKit/Core/GGMLDequant.swift:125-428) bit for bit, so every product is written
// with explicit single-rounding intrinsics in the reference's order of operations and nothing
// here may be compiled with fast-math.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "ggml_tables.h"
#include "iq2xs_tables.h"
#include "ishi_ptx.cuh"

namespace ishi {

// codebooks (Sources/IshizukiKit/Core/GGMLTables.swift:26-1137), byte j of an entry = value j
static __device__ const uint64_t d_iq2xxs_grid[256] = {ISHI_IQ2_XXS_GRID_LIST};
static __device__ const uint16_t d_iq2xs_codes[512] = {ISHI_IQ2XS_CODES_LIST};
static __device__ const uint64_t d_iq2s_grid[1024] = {ISHI_IQ2_S_GRID_LIST};
static __device__ const uint32_t d_iq3xxs_grid[256] = {ISHI_IQ3_XXS_GRID_LIST};
static __device__ const uint32_t d_iq3s_grid[512] = {ISHI_IQ3_S_GRID_LIST};
static __device__ const uint64_t d_iq1s_grid[2048] = {ISHI_IQ1_S_GRID_LIST};
static __device__ const int8_t d_kvalues_iq4nl[16] = {ISHI_IQ4NL_VALUES_LIST};

// GGMLType.typeSize (Sources/IshizukiKit/Config/GGUFFile.swift:44-80); 0: no decoder here
__host__ __device__ constexpr int ggml_type_bytes(int type) {
  return type == 10 ? 84 : type == 12 ? 144 : type == 14 ? 210 : type == 16 ? 66 : type == 17 ? 74 : type == 18 ? 98
       : type == 19 ? 50 : type == 21 ? 110 : type == 22 ? 82 : type == 23 ? 136 : type == 29 ? 56 : 0;
}

__device__ __forceinline__ float rd_half(const uint8_t *p) {
  return half_bits_to_float((uint32_t)p[0] | ((uint32_t)p[1] << 8));
}
__device__ __forceinline__ uint32_t rd_u16(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8); }
__device__ __forceinline__ uint32_t rd_u32(const uint8_t *p) { return rd_u16(p) | (rd_u16(p + 2) << 16); }
// the i-quants' sign byte of 7-bit index i: i with bit 7 = parity(i) (GGMLTables.swift:15-24)
__device__ __forceinline__ uint32_t ksigns(uint32_t i) { return i | ((__popc(i) & 1u) << 7); }
__device__ __forceinline__ float sign_of(uint32_t signs, int j) { return ((signs >> j) & 1u) ? -1.0f : 1.0f; }

// Q2_K (GGMLDequant.swift:125-150): scale | min << 4 bytes @0, 2-bit codes @16, d @80, dmin @82
__device__ __forceinline__ void decode8_q2k(const uint8_t *b, int lane, float (&w)[8]) {
  const int half = lane >> 4, sh = (lane >> 2) & 3, l16 = (lane >> 1) & 1, l0 = 8 * (lane & 1);
  const uint32_t sc = b[half * 8 + sh * 2 + l16];
  const float dl = __fmul_rn(rd_half(b + 80), (float)(sc & 0xfu)), ml = __fmul_rn(rd_half(b + 82), (float)(sc >> 4));
  const uint8_t *q = b + 16 + half * 32 + l16 * 16 + l0;
#pragma unroll
  for (int e = 0; e < 8; ++e) w[e] = __fsub_rn(__fmul_rn(dl, (float)((q[e] >> (2 * sh)) & 3u)), ml);
}

// Q4_K (GGMLDequant.swift:187-220)
__device__ __forceinline__ void decode8_q4k(const uint8_t *b, int lane, float (&w)[8]) {
  const int j = lane >> 3;           // 64-weight chunk
  const int hi = (lane >> 2) & 1;    // second 32 of the chunk: high nibbles
  const int i = 2 * j + hi;          // sub-block
  const uint8_t *q = b + 4;
  uint32_t sc, m;
  if (i < 4) {
    sc = q[i] & 63u;
    m = q[i + 4] & 63u;
  } else {
    sc = (q[i + 4] & 0xfu) | ((uint32_t)(q[i - 4] >> 6) << 4);
    m = (uint32_t)(q[i + 4] >> 4) | ((uint32_t)(q[i] >> 6) << 4);
  }
  const float dl = __fmul_rn(rd_half(b), (float)sc);
  const float ml = __fmul_rn(rd_half(b + 2), (float)m);
  const uint8_t *qs = b + 16 + 32 * j + 8 * (lane & 3);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const uint32_t v = hi ? (uint32_t)(qs[e] >> 4) : (uint32_t)(qs[e] & 0xfu);
    w[e] = __fsub_rn(__fmul_rn(dl, (float)v), ml);
  }
}

// Q6_K (GGMLDequant.swift:154-185)
__device__ __forceinline__ void decode8_q6k(const uint8_t *b, int lane, float (&w)[8]) {
  const int half = lane >> 4;          // 128-weight half
  const int run = (lane >> 2) & 3;     // which of the four 32-weight runs of the half
  const int l0 = 8 * (lane & 3);       // offset inside the run
  const uint8_t *ql = b + 64 * half + 32 * (run & 1) + l0;
  const uint8_t *qh = b + 128 + 32 * half + l0;
  const int8_t scale = ((const int8_t *)b)[192 + 8 * half + 2 * run + l0 / 16];
  const float dl = __fmul_rn(rd_half(b + 208), (float)scale);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const uint32_t nib = run < 2 ? (uint32_t)(ql[e] & 0xfu) : (uint32_t)(ql[e] >> 4);
    const int qv = (int)(nib | (((uint32_t)(qh[e] >> (2 * run)) & 3u) << 4)) - 32;
    w[e] = __fmul_rn(dl, (float)qv);
  }
}

// IQ4_XS (GGMLDequant.swift:222-241): d @0, scales_h @2, scales_l @4, nibbles @8
__device__ __forceinline__ void decode8_iq4xs(const uint8_t *b, int lane, float (&w)[8]) {
  const int ib = lane >> 2, pos = 8 * (lane & 3);
  const int low = (b[4 + ib / 2] >> (4 * (ib % 2))) & 0xf;
  const int high = (int)((rd_u16(b + 2) >> (2 * ib)) & 3u) << 4;
  const float dl = __fmul_rn(rd_half(b), (float)((low | high) - 32));
  const uint8_t *qs = b + 8 + 16 * ib + (pos & 15);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const uint32_t q = pos < 16 ? (uint32_t)(qs[e] & 0xfu) : (uint32_t)(qs[e] >> 4);
    w[e] = __fmul_rn(dl, (float)d_kvalues_iq4nl[q]);
  }
}

// IQ2_XXS (GGMLDequant.swift:243-262)
__device__ __forceinline__ void decode8_iq2xxs(const uint8_t *b, int lane, float (&w)[8]) {
  const int ib = lane >> 2, l = lane & 3;
  const uint32_t aux1 = rd_u32(b + 2 + 8 * ib), aux2 = rd_u32(b + 6 + 8 * ib);
  const float db = __fmul_rn(__fmul_rn(rd_half(b), 0.5f + (float)(aux2 >> 28)), 0.25f);
  const uint64_t e64 = d_iq2xxs_grid[(aux1 >> (8 * l)) & 0xffu];
  const uint32_t signs = ksigns((aux2 >> (7 * l)) & 127u);
#pragma unroll
  for (int e = 0; e < 8; ++e) w[e] = __fmul_rn(__fmul_rn(db, (float)((e64 >> (8 * e)) & 0xffull)), sign_of(signs, e));
}

// IQ2_XS (GGMLDequant.swift:264-285)
__device__ __forceinline__ void decode8_iq2xs(const uint8_t *b, int lane, float (&w)[8]) {
  const int ib = lane >> 2, l = lane & 3;
  const uint32_t sbyte = b[66 + ib];
  const uint32_t s = l < 2 ? (sbyte & 0xfu) : (sbyte >> 4);
  const float db = __fmul_rn(__fmul_rn(rd_half(b), 0.5f + (float)s), 0.25f);
  const uint32_t q = rd_u16(b + 2 + 2 * lane);
  const uint32_t codes = d_iq2xs_codes[q & 511u];
  const uint32_t signs = ksigns(q >> 9);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const uint32_t c = (codes >> (2 * e)) & 3u;
    const float gv = c == 0 ? (float)ISHI_IQ2XS_VALUE0 : (c == 1 ? (float)ISHI_IQ2XS_VALUE1 : (float)ISHI_IQ2XS_VALUE2);
    w[e] = __fmul_rn(__fmul_rn(db, gv), sign_of(signs, e));
  }
}

// IQ2_S (GGMLDequant.swift:287-311): d @0, index bytes @2, sign bytes @34, qh @66, scales @74
__device__ __forceinline__ void decode8_iq2s(const uint8_t *b, int lane, float (&w)[8]) {
  const int ib = lane >> 2, l = lane & 3;
  const uint32_t scale = b[74 + ib];
  const float db = __fmul_rn(__fmul_rn(rd_half(b), 0.5f + (float)(l < 2 ? (scale & 0xfu) : (scale >> 4))), 0.25f);
  const uint32_t idx = (uint32_t)b[2 + 4 * ib + l] | (((uint32_t)b[66 + ib] << (8 - 2 * l)) & 0x300u);
  const uint64_t e64 = d_iq2s_grid[idx];
  const uint32_t signs = b[34 + 4 * ib + l];
#pragma unroll
  for (int e = 0; e < 8; ++e) w[e] = __fmul_rn(__fmul_rn(db, (float)((e64 >> (8 * e)) & 0xffull)), sign_of(signs, e));
}

// IQ3_XXS (GGMLDequant.swift:313-335): d @0, index bytes @2, signs and scales @66
__device__ __forceinline__ void decode8_iq3xxs(const uint8_t *b, int lane, float (&w)[8]) {
  const int ib = lane >> 2, l = lane & 3;
  const uint32_t aux = rd_u32(b + 66 + 4 * ib);
  const float db = __fmul_rn(__fmul_rn(rd_half(b), 0.5f + (float)(aux >> 28)), 0.5f);
  const uint32_t signs = ksigns((aux >> (7 * l)) & 127u);
  const uint32_t g1 = d_iq3xxs_grid[b[2 + 8 * ib + 2 * l]], g2 = d_iq3xxs_grid[b[2 + 8 * ib + 2 * l + 1]];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    w[e] = __fmul_rn(__fmul_rn(db, (float)((g1 >> (8 * e)) & 0xffu)), sign_of(signs, e));
    w[4 + e] = __fmul_rn(__fmul_rn(db, (float)((g2 >> (8 * e)) & 0xffu)), sign_of(signs, e + 4));
  }
}

// IQ3_S (GGMLDequant.swift:337-374): d @0, index bytes @2, qh @66, sign bytes @74, scales @106
__device__ __forceinline__ void decode8_iq3s(const uint8_t *b, int lane, float (&w)[8]) {
  const int ib = lane >> 2, l = lane & 3;
  const uint32_t scale = b[106 + ib / 2];
  const float db = __fmul_rn(rd_half(b), (float)(1 + 2 * (int)((ib & 1) ? (scale >> 4) : (scale & 0xfu))));
  const uint32_t qh = b[66 + ib];
  const uint8_t *qs = b + 2 + 8 * ib;
  const uint32_t g1 = d_iq3s_grid[(uint32_t)qs[2 * l] | ((qh << (8 - 2 * l)) & 256u)];
  const uint32_t g2 = d_iq3s_grid[(uint32_t)qs[2 * l + 1] | ((qh << (7 - 2 * l)) & 256u)];
  const uint32_t signs = b[74 + 4 * ib + l];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    w[e] = __fmul_rn(__fmul_rn(db, (float)((g1 >> (8 * e)) & 0xffu)), sign_of(signs, e));
    w[4 + e] = __fmul_rn(__fmul_rn(db, (float)((g2 >> (8 * e)) & 0xffu)), sign_of(signs, e + 4));
  }
}

// the 2048-entry grid of IQ1_S and IQ1_M holds signed bytes out of {-1, 0, 1}
__device__ __forceinline__ float iq1_value(uint64_t e64, int j) { return (float)(int8_t)((e64 >> (8 * j)) & 0xffull); }

// IQ1_S (GGMLDequant.swift:376-395): d @0, index bytes @2, qh words @34
__device__ __forceinline__ void decode8_iq1s(const uint8_t *b, int lane, float (&w)[8]) {
  const int ib = lane >> 2, l = lane & 3;
  const uint32_t qh = rd_u16(b + 34 + 2 * ib);
  const float dl = __fmul_rn(rd_half(b), (float)(2 * (int)((qh >> 12) & 7u) + 1));
  const float delta = (qh & 0x8000u) ? -0.125f : 0.125f;
  const uint64_t e64 = d_iq1s_grid[(uint32_t)b[2 + 4 * ib + l] | (((qh >> (3 * l)) & 7u) << 8)];
#pragma unroll
  for (int e = 0; e < 8; ++e) w[e] = __fmul_rn(dl, __fadd_rn(iq1_value(e64, e), delta));
}

// IQ1_M (GGMLDequant.swift:397-428): index bytes @0, qh @32, four scale words @48 whose top
// nibbles spell the fp16 block scale
__device__ __forceinline__ void decode8_iq1m(const uint8_t *b, int lane, float (&w)[8]) {
  const int ib = lane >> 2, l = lane & 3;
  const uint32_t s0 = rd_u16(b + 48), s1 = rd_u16(b + 50), s2 = rd_u16(b + 52), s3 = rd_u16(b + 54);
  const float d = half_bits_to_float((s0 >> 12) | ((s1 >> 8) & 0x00f0u) | ((s2 >> 4) & 0x0f00u) | (s3 & 0xf000u));
  const uint32_t word = rd_u16(b + 48 + 2 * (ib / 2));
  const int shift = 6 * (ib % 2) + (l < 2 ? 0 : 3);
  const float dl = __fmul_rn(d, (float)(2 * (int)((word >> shift) & 7u) + 1));
  const uint32_t qh = b[32 + 2 * ib + (l >> 1)];
  const uint32_t idx = (uint32_t)b[4 * ib + l] | (((l & 1) ? (qh << 4) : (qh << 8)) & 0x700u);
  const float delta = (qh & ((l & 1) ? 0x80u : 0x08u)) ? -0.125f : 0.125f;
  const uint64_t e64 = d_iq1s_grid[idx];
#pragma unroll
  for (int e = 0; e < 8; ++e) w[e] = __fmul_rn(dl, __fadd_rn(iq1_value(e64, e), delta));
}

template <int TYPE>
__device__ __forceinline__ void decode8(const uint8_t *b, int lane, float (&w)[8]) {
  if (TYPE == 10) decode8_q2k(b, lane, w);
  else if (TYPE == 12) decode8_q4k(b, lane, w);
  else if (TYPE == 14) decode8_q6k(b, lane, w);
  else if (TYPE == 16) decode8_iq2xxs(b, lane, w);
  else if (TYPE == 17) decode8_iq2xs(b, lane, w);
  else if (TYPE == 18) decode8_iq3xxs(b, lane, w);
  else if (TYPE == 19) decode8_iq1s(b, lane, w);
  else if (TYPE == 21) decode8_iq3s(b, lane, w);
  else if (TYPE == 22) decode8_iq2s(b, lane, w);
  else if (TYPE == 23) decode8_iq4xs(b, lane, w);
  else decode8_iq1m(b, lane, w);
}

}  // namespace ishi
