/* CPU oracle for the speculative-verify quantized matmul. TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's algorithm for this path, used as the checker in
 * tests/, in the smoke check and as the timed CPU baseline of bench.py. Nothing in the product
 * package may call into this file: the product path is the CUDA library and fails without it.
 *
 * What each function follows in the reference (paths inside the reference project):
 *   - oracle_dequant_q4k   Sources/IshizukiKit/Core/GGMLDequant.swift:187-220
 *   - oracle_dequant_q6k   Sources/IshizukiKit/Core/GGMLDequant.swift:154-185
 *   - oracle_dequant_iq2xs Sources/IshizukiKit/Core/GGMLDequant.swift:264-285, sign table
 *                          Sources/IshizukiKit/Core/GGMLTables.swift:11-24
 *   - oracle_dequant_q2k, _iq4xs, _iq2xxs, _iq2s, _iq3xxs, _iq3s, _iq1s, _iq1m
 *                          Sources/IshizukiKit/Core/GGMLDequant.swift:125-150, 222-262, 287-428,
 *                          codebooks Sources/IshizukiKit/Core/GGMLTables.swift:26-1137
 *   - oracle_affine_dequant Sources/IshizukiKit/Core/VerifyMatmul.swift:282-287 (code i of a
 *                          row at bit i*bits of the row's word stream, w = float(code)*s + b)
 *                          and Sources/IshizukiKit/Quantize/WeightedAffineQuantizer.swift:142-161
 *   - oracle_hadamard_rotate Sources/IshizukiKit/Core/Hadamard.swift:8-23 and
 *                          Sources/IshizukiKit/Core/FusedHadamard.swift:54-78
 *   - oracle_matmul        the "expand the weight and multiply" definition the reference's tests
 *                          compare against (Tests/IshizukiKitTests/GGMLKernelTests.swift:111-140,
 *                          Tests/IshizukiKitTests/VerifyMatmulTests.swift:31-45)
 *
 * Parity pin: the eleven dequantizers reproduce ggml's own to_float bit for bit on the
 * reference's fixture Tests/IshizukiKitTests/Fixtures/ggml-reference.bin (types 10, 12, 14,
 * 16, 17, 18, 19, 21, 22, 23, 29);
 * the rotation reproduces Tests/Golden/hadamard_golden.safetensors case1. The affine formula
 * has no stored vector in the reference (its tests compare against MLX live): that part is
 * pinned by the formula only.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../ishizuki_b200/csrc/ggml_tables.h"
#include "../ishizuki_b200/csrc/iq2xs_tables.h"

/* ---- scalar helpers ---------------------------------------------------------------------- */

static float half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do {
        man <<= 1;
        e++;
      } while ((man & 0x400u) == 0);
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* Round to nearest even, as a GPU store of an fp32 value into an fp16 array does. */
static uint16_t float_to_half(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t absx = x & 0x7fffffffu;
  if (absx >= 0x7f800000u) { /* inf / nan */
    return (uint16_t)(sign | 0x7c00u | (absx > 0x7f800000u ? 0x200u | ((absx >> 13) & 0x3ffu) : 0));
  }
  if (absx >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7c00u);
  }
  if (absx < 0x33000001u) { /* below half the smallest subnormal */
    return (uint16_t)sign;
  }
  int32_t e = (int32_t)(absx >> 23) - 127;
  uint32_t m = (absx & 0x7fffffu) | 0x800000u;
  int shift;
  uint32_t base;
  if (e < -14) {
    shift = 13 + (-14 - e);
    base = 0;
  } else {
    shift = 13;
    base = (uint32_t)(e + 15) << 10;
    m &= 0x7fffffu;
  }
  uint32_t q = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1u);
  uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (q & 1u))) q++;
  return (uint16_t)(sign | (base + q));
}

static float bf16_to_float(uint16_t b) {
  uint32_t bits = (uint32_t)b << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

uint16_t oracle_float_to_half(float f) { return float_to_half(f); }
float oracle_half_to_float(uint16_t h) { return half_to_float(h); }

/* ---- GGUF block dequantizers -------------------------------------------------------------- */

/* Q4_K, 144 bytes per 256 weights: d f16 @0, dmin f16 @2, twelve bytes of 6-bit (scale, min)
 * pairs @4, 128 bytes of nibbles @16. Reference: GGMLDequant.swift:187-220. */
void oracle_dequant_q4k(const uint8_t *blocks, int64_t nblocks, float *y) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t *p = blocks + b * 144;
    const float d = half_to_float(rd16(p));
    const float dmin = half_to_float(rd16(p + 2));
    const uint8_t *q = p + 4;
    float *out = y + b * 256;
    int pair = 0;
    for (int j = 0; j < 256; j += 64) {
      float dl[2], ml[2];
      for (int h = 0; h < 2; ++h) {
        const int i = pair + h;
        uint8_t sc, m;
        if (i < 4) {
          sc = q[i] & 63;
          m = q[i + 4] & 63;
        } else {
          sc = (uint8_t)((q[i + 4] & 0xf) | ((q[i - 4] >> 6) << 4));
          m = (uint8_t)((q[i + 4] >> 4) | ((q[i] >> 6) << 4));
        }
        dl[h] = d * (float)sc;
        ml[h] = dmin * (float)m;
      }
      const uint8_t *qs = p + 16 + j / 2;
      for (int l = 0; l < 32; ++l) {
        out[l] = dl[0] * (float)(qs[l] & 0xf) - ml[0];
        out[32 + l] = dl[1] * (float)(qs[l] >> 4) - ml[1];
      }
      out += 64;
      pair += 2;
    }
  }
}

/* Q6_K, 210 bytes: ql[128] @0, qh[64] @128, int8 scales[16] @192, d f16 @208.
 * Reference: GGMLDequant.swift:154-185; the product is (d * scale) * (q - 32). */
void oracle_dequant_q6k(const uint8_t *blocks, int64_t nblocks, float *y) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t *p = blocks + b * 210;
    const float d = half_to_float(rd16(p + 208));
    float *out = y + b * 256;
    const uint8_t *ql = p;
    const uint8_t *qh = p + 128;
    const int8_t *sc = (const int8_t *)(p + 192);
    for (int half = 0; half < 2; ++half) {
      for (int l = 0; l < 32; ++l) {
        const uint8_t hb = qh[l];
        const int q1 = (ql[l] & 0xf) | (((hb >> 0) & 3) << 4);
        const int q2 = (ql[32 + l] & 0xf) | (((hb >> 2) & 3) << 4);
        const int q3 = (ql[l] >> 4) | (((hb >> 4) & 3) << 4);
        const int q4 = (ql[32 + l] >> 4) | (((hb >> 6) & 3) << 4);
        const int g = l / 16;
        out[l] = d * (float)sc[g + 0] * (float)(q1 - 32);
        out[32 + l] = d * (float)sc[g + 2] * (float)(q2 - 32);
        out[64 + l] = d * (float)sc[g + 4] * (float)(q3 - 32);
        out[96 + l] = d * (float)sc[g + 6] * (float)(q4 - 32);
      }
      out += 128;
      ql += 64;
      qh += 32;
      sc += 8;
    }
  }
}

/* The 128-entry sign table of the i-quants: entry i is i with bit 7 set when i has an odd
 * number of one bits (GGMLTables.swift:15-24 lists the same 128 values). */
static uint8_t ksigns(int i) { return (uint8_t)(i | ((__builtin_popcount((unsigned)i) & 1) << 7)); }

static const float iq2xs_value[3] = {ISHI_IQ2XS_VALUE0, ISHI_IQ2XS_VALUE1, ISHI_IQ2XS_VALUE2};

/* IQ2_XS, 74 bytes: d f16 @0, 32 x u16 @2 (bits 0-8 grid index, 9-15 sign index), eight scale
 * bytes @66 (low nibble first sixteen weights of a 32-group, high nibble the second sixteen).
 * Reference: GGMLDequant.swift:264-285. */
void oracle_dequant_iq2xs(const uint8_t *blocks, int64_t nblocks, float *y) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t *p = blocks + b * 74;
    const float d = half_to_float(rd16(p));
    float *out = y + b * 256;
    for (int ib = 0; ib < 8; ++ib) {
      const uint8_t s = p[66 + ib];
      const float db[2] = {d * (0.5f + (float)(s & 0xf)) * 0.25f, d * (0.5f + (float)(s >> 4)) * 0.25f};
      for (int l = 0; l < 4; ++l) {
        const uint16_t q = rd16(p + 2 + 2 * (4 * ib + l));
        const uint16_t codes = ISHI_IQ2XS_CODES[q & 511];
        const uint8_t signs = ksigns(q >> 9);
        for (int j = 0; j < 8; ++j) {
          const float g = iq2xs_value[(codes >> (2 * j)) & 3];
          out[j] = db[l / 2] * g * ((signs >> j) & 1 ? -1.0f : 1.0f);
        }
        out += 8;
      }
    }
  }
}

static uint32_t rd32(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }

static const uint64_t iq2xxs_grid[256] = {ISHI_IQ2_XXS_GRID_LIST};
static const uint64_t iq2s_grid[1024] = {ISHI_IQ2_S_GRID_LIST};
static const uint32_t iq3xxs_grid[256] = {ISHI_IQ3_XXS_GRID_LIST};
static const uint32_t iq3s_grid[512] = {ISHI_IQ3_S_GRID_LIST};
static const uint64_t iq1s_grid[2048] = {ISHI_IQ1_S_GRID_LIST};
static const int8_t kvalues_iq4nl[16] = {ISHI_IQ4NL_VALUES_LIST};

static float grid_byte64(uint64_t e, int j) { return (float)((e >> (8 * j)) & 0xff); }
static float grid_sbyte64(uint64_t e, int j) { return (float)(int8_t)((e >> (8 * j)) & 0xff); }
static float grid_byte32(uint32_t e, int j) { return (float)((e >> (8 * j)) & 0xff); }
static float sign_flip(uint8_t signs, int j) { return (signs >> j) & 1 ? -1.0f : 1.0f; }

/* Q2_K, 84 bytes: sixteen (scale | min << 4) bytes @0, 64 bytes of 2-bit codes @16, d f16 @80,
 * dmin f16 @82. Reference: GGMLDequant.swift:125-150. */
void oracle_dequant_q2k(const uint8_t *blocks, int64_t nblocks, float *y) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t *p = blocks + b * 84;
    const float d = half_to_float(rd16(p + 80)), dmin = half_to_float(rd16(p + 82));
    float *out = y + b * 256;
    int scale = 0;
    for (int n = 0; n < 256; n += 128) {
      const uint8_t *q = p + 16 + n / 4;
      for (int shift = 0; shift < 8; shift += 2) {
        for (int lane = 0; lane < 2; ++lane) {
          const uint8_t sc = p[scale++];
          const float dl = d * (float)(sc & 0xf), ml = dmin * (float)(sc >> 4);
          for (int l = 0; l < 16; ++l) *out++ = dl * (float)((q[16 * lane + l] >> shift) & 3) - ml;
        }
      }
    }
  }
}

/* IQ4_XS, 136 bytes: d f16 @0, scales_h u16 @2, four scales_l bytes @4, 128 nibble bytes @8;
 * values through the sixteen-entry non-linear table. Reference: GGMLDequant.swift:222-241. */
void oracle_dequant_iq4xs(const uint8_t *blocks, int64_t nblocks, float *y) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t *p = blocks + b * 136;
    const float d = half_to_float(rd16(p));
    const uint16_t scales_h = rd16(p + 2);
    float *out = y + b * 256;
    for (int ib = 0; ib < 8; ++ib) {
      const int low = (p[4 + ib / 2] >> (4 * (ib % 2))) & 0xf;
      const int high = ((scales_h >> (2 * ib)) & 3) << 4;
      const float dl = d * (float)((low | high) - 32);
      const uint8_t *qs = p + 8 + 16 * ib;
      for (int j = 0; j < 16; ++j) {
        out[j] = dl * (float)kvalues_iq4nl[qs[j] & 0xf];
        out[16 + j] = dl * (float)kvalues_iq4nl[qs[j] >> 4];
      }
      out += 32;
    }
  }
}

/* IQ2_XXS, 66 bytes: d f16 @0, per 32 weights two u32 @2: four grid indices, then four 7-bit
 * sign indices and a 4-bit scale. Reference: GGMLDequant.swift:243-262. */
void oracle_dequant_iq2xxs(const uint8_t *blocks, int64_t nblocks, float *y) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t *p = blocks + b * 66;
    const float d = half_to_float(rd16(p));
    float *out = y + b * 256;
    for (int ib = 0; ib < 8; ++ib) {
      const uint32_t aux1 = rd32(p + 2 + 8 * ib), aux2 = rd32(p + 6 + 8 * ib);
      const float db = d * (0.5f + (float)(aux2 >> 28)) * 0.25f;
      for (int l = 0; l < 4; ++l) {
        const uint64_t e = iq2xxs_grid[(aux1 >> (8 * l)) & 0xff];
        const uint8_t signs = ksigns((aux2 >> (7 * l)) & 127);
        for (int j = 0; j < 8; ++j) out[j] = db * grid_byte64(e, j) * sign_flip(signs, j);
        out += 8;
      }
    }
  }
}

/* IQ2_S, 82 bytes: d f16 @0, 32 index bytes @2, 32 sign bytes @34, 8 qh bytes @66, 8 scale
 * bytes @74. Reference: GGMLDequant.swift:287-311. */
void oracle_dequant_iq2s(const uint8_t *blocks, int64_t nblocks, float *y) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t *p = blocks + b * 82;
    const float d = half_to_float(rd16(p));
    float *out = y + b * 256;
    for (int ib = 0; ib < 8; ++ib) {
      const uint8_t scale = p[74 + ib];
      const float db[2] = {d * (0.5f + (float)(scale & 0xf)) * 0.25f, d * (0.5f + (float)(scale >> 4)) * 0.25f};
      const int qh = p[66 + ib];
      for (int l = 0; l < 4; ++l) {
        const int low = p[2 + 4 * ib + l];
        const int high = (qh << (8 - 2 * l)) & 0x300;
        const uint64_t e = iq2s_grid[low | high];
        const uint8_t signs = p[34 + 4 * ib + l];
        for (int j = 0; j < 8; ++j) out[j] = db[l / 2] * grid_byte64(e, j) * sign_flip(signs, j);
        out += 8;
      }
    }
  }
}

/* IQ3_XXS, 98 bytes: d f16 @0, 64 index bytes @2, per 32 weights one u32 @66 (four 7-bit sign
 * indices and a 4-bit scale). Reference: GGMLDequant.swift:313-335. */
void oracle_dequant_iq3xxs(const uint8_t *blocks, int64_t nblocks, float *y) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t *p = blocks + b * 98;
    const float d = half_to_float(rd16(p));
    float *out = y + b * 256;
    for (int ib = 0; ib < 8; ++ib) {
      const uint32_t aux = rd32(p + 66 + 4 * ib);
      const float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
      for (int l = 0; l < 4; ++l) {
        const uint8_t signs = ksigns((aux >> (7 * l)) & 127);
        const uint32_t g1 = iq3xxs_grid[p[2 + 8 * ib + 2 * l]], g2 = iq3xxs_grid[p[2 + 8 * ib + 2 * l + 1]];
        for (int j = 0; j < 4; ++j) {
          out[j] = db * grid_byte32(g1, j) * sign_flip(signs, j);
          out[4 + j] = db * grid_byte32(g2, j) * sign_flip(signs, j + 4);
        }
        out += 8;
      }
    }
  }
}

/* IQ3_S, 110 bytes: d f16 @0, 64 index bytes @2, 8 qh bytes @66, 32 sign bytes @74, 4 scale
 * bytes @106. Reference: GGMLDequant.swift:337-374. */
void oracle_dequant_iq3s(const uint8_t *blocks, int64_t nblocks, float *y) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t *p = blocks + b * 110;
    const float d = half_to_float(rd16(p));
    float *out = y + b * 256;
    for (int pair = 0; pair < 8; pair += 2) {
      const uint8_t scale = p[106 + pair / 2];
      const float db[2] = {d * (float)(1 + 2 * (scale & 0xf)), d * (float)(1 + 2 * (scale >> 4))};
      for (int group = 0; group < 2; ++group) {
        const int qh = p[66 + pair + group];
        const uint8_t *qs = p + 2 + 8 * (pair + group);
        const uint8_t *signs = p + 74 + 4 * (pair + group);
        for (int l = 0; l < 4; ++l) {
          const uint32_t g1 = iq3s_grid[qs[2 * l] | ((qh << (8 - 2 * l)) & 256)];
          const uint32_t g2 = iq3s_grid[qs[2 * l + 1] | ((qh << (7 - 2 * l)) & 256)];
          for (int j = 0; j < 4; ++j) {
            out[j] = db[group] * grid_byte32(g1, j) * sign_flip(signs[l], j);
            out[4 + j] = db[group] * grid_byte32(g2, j) * sign_flip(signs[l], j + 4);
          }
          out += 8;
        }
      }
    }
  }
}

/* IQ1_S, 50 bytes: d f16 @0, 32 index bytes @2, eight u16 @34 (four 3-bit index extensions, a
 * 3-bit scale, a delta sign). Reference: GGMLDequant.swift:376-395. */
void oracle_dequant_iq1s(const uint8_t *blocks, int64_t nblocks, float *y) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t *p = blocks + b * 50;
    const float d = half_to_float(rd16(p));
    float *out = y + b * 256;
    for (int ib = 0; ib < 8; ++ib) {
      const uint16_t qh = rd16(p + 34 + 2 * ib);
      const float dl = d * (float)(2 * ((qh >> 12) & 7) + 1);
      const float delta = (qh & 0x8000) ? -0.125f : 0.125f;
      for (int l = 0; l < 4; ++l) {
        const uint64_t e = iq1s_grid[p[2 + 4 * ib + l] | (((qh >> (3 * l)) & 7) << 8)];
        for (int j = 0; j < 8; ++j) out[j] = dl * (grid_sbyte64(e, j) + delta);
        out += 8;
      }
    }
  }
}

/* IQ1_M, 56 bytes: 32 index bytes @0, 16 qh bytes @32, four u16 @48 whose top nibbles spell the
 * fp16 block scale and whose low 12 bits hold four 3-bit scales. Reference:
 * GGMLDequant.swift:397-428. */
void oracle_dequant_iq1m(const uint8_t *blocks, int64_t nblocks, float *y) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t *p = blocks + b * 56;
    uint16_t sc[4];
    for (int i = 0; i < 4; ++i) sc[i] = rd16(p + 48 + 2 * i);
    const uint16_t packed = (uint16_t)((sc[0] >> 12) | ((sc[1] >> 8) & 0x00f0) | ((sc[2] >> 4) & 0x0f00) | (sc[3] & 0xf000));
    const float d = half_to_float(packed);
    float *out = y + b * 256;
    for (int ib = 0; ib < 8; ++ib) {
      const uint16_t word = sc[ib / 2];
      const int shift = 6 * (ib % 2);
      const float dl1 = d * (float)(2 * ((word >> shift) & 7) + 1);
      const float dl2 = d * (float)(2 * ((word >> (shift + 3)) & 7) + 1);
      const int qh0 = p[32 + 2 * ib], qh1 = p[32 + 2 * ib + 1];
      const int index[4] = {p[4 * ib] | ((qh0 << 8) & 0x700), p[4 * ib + 1] | ((qh0 << 4) & 0x700),
                            p[4 * ib + 2] | ((qh1 << 8) & 0x700), p[4 * ib + 3] | ((qh1 << 4) & 0x700)};
      const float delta[4] = {(qh0 & 0x08) ? -0.125f : 0.125f, (qh0 & 0x80) ? -0.125f : 0.125f,
                              (qh1 & 0x08) ? -0.125f : 0.125f, (qh1 & 0x80) ? -0.125f : 0.125f};
      for (int l = 0; l < 4; ++l) {
        const float dl = l < 2 ? dl1 : dl2;
        const uint64_t e = iq1s_grid[index[l]];
        for (int j = 0; j < 8; ++j) out[j] = dl * (grid_sbyte64(e, j) + delta[l]);
        out += 8;
      }
    }
  }
}

/* GGML type ids as in Sources/IshizukiKit/Config/GGUFFile.swift:13-44, block sizes as in
 * :44-80 (pinned by Tests/IshizukiKitTests/GGUFTests.swift:17-35). */
enum {
  GGML_Q2_K = 10, GGML_Q4_K = 12, GGML_Q6_K = 14, GGML_IQ2_XXS = 16, GGML_IQ2_XS = 17, GGML_IQ3_XXS = 18,
  GGML_IQ1_S = 19, GGML_IQ3_S = 21, GGML_IQ2_S = 22, GGML_IQ4_XS = 23, GGML_IQ1_M = 29
};

int oracle_type_size(int type) {
  switch (type) {
    case GGML_Q2_K: return 84;
    case GGML_Q4_K: return 144;
    case GGML_Q6_K: return 210;
    case GGML_IQ2_XXS: return 66;
    case GGML_IQ2_XS: return 74;
    case GGML_IQ3_XXS: return 98;
    case GGML_IQ1_S: return 50;
    case GGML_IQ3_S: return 110;
    case GGML_IQ2_S: return 82;
    case GGML_IQ4_XS: return 136;
    case GGML_IQ1_M: return 56;
    default: return 0;
  }
}

int oracle_dequant(int type, const uint8_t *blocks, int64_t nblocks, float *y) {
  switch (type) {
    case GGML_Q2_K: oracle_dequant_q2k(blocks, nblocks, y); return 0;
    case GGML_Q4_K: oracle_dequant_q4k(blocks, nblocks, y); return 0;
    case GGML_Q6_K: oracle_dequant_q6k(blocks, nblocks, y); return 0;
    case GGML_IQ2_XXS: oracle_dequant_iq2xxs(blocks, nblocks, y); return 0;
    case GGML_IQ2_XS: oracle_dequant_iq2xs(blocks, nblocks, y); return 0;
    case GGML_IQ3_XXS: oracle_dequant_iq3xxs(blocks, nblocks, y); return 0;
    case GGML_IQ1_S: oracle_dequant_iq1s(blocks, nblocks, y); return 0;
    case GGML_IQ3_S: oracle_dequant_iq3s(blocks, nblocks, y); return 0;
    case GGML_IQ2_S: oracle_dequant_iq2s(blocks, nblocks, y); return 0;
    case GGML_IQ4_XS: oracle_dequant_iq4xs(blocks, nblocks, y); return 0;
    case GGML_IQ1_M: oracle_dequant_iq1m(blocks, nblocks, y); return 0;
    default: return -1;
  }
}

/* ---- MLX affine packs --------------------------------------------------------------------- */

/* scale_dtype: 0 = f16, 1 = bf16, 2 = f32 */
static float load_scale(const void *base, int64_t i, int dtype) {
  switch (dtype) {
    case 0: return half_to_float(((const uint16_t *)base)[i]);
    case 1: return bf16_to_float(((const uint16_t *)base)[i]);
    default: return ((const float *)base)[i];
  }
}

/* One row of an affine pack to floats: code i sits at bit i*bits of the row's little-endian
 * word stream (a code may straddle two words for widths that do not divide 32), and
 * w = float(code) * scale + bias with the group's scale and bias. */
static void affine_row(const uint32_t *w, int64_t K, int bits, int gs, const void *scales,
                       const void *biases, int sdt, int64_t srow, float *out) {
  const uint32_t mask = (1u << bits) - 1u;
  for (int64_t k = 0; k < K; ++k) {
    const int64_t bit = k * bits;
    const int64_t word = bit >> 5;
    const int off = (int)(bit & 31);
    uint32_t v = w[word] >> off;
    if (off + bits > 32) v |= w[word + 1] << (32 - off);
    const float s = load_scale(scales, srow + k / gs, sdt);
    const float b = load_scale(biases, srow + k / gs, sdt);
    out[k] = (float)(v & mask) * s + b;
  }
}

int oracle_affine_dequant(const uint32_t *w, const void *scales, const void *biases,
                          int scale_dtype, int64_t N, int64_t K, int bits, int group_size,
                          float *y) {
  if (bits < 2 || bits > 8 || K % group_size != 0 || (K * bits) % 32 != 0) return -1;
  const int64_t words = K * bits / 32;
  const int64_t groups = K / group_size;
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n) {
    affine_row(w + n * words, K, bits, group_size, scales, biases, scale_dtype, n * groups,
               y + n * K);
  }
  return 0;
}

/* ---- Hadamard rotation --------------------------------------------------------------------- */

/* x' = WHT_block(x * signs) / sqrt(block) along the last axis in fp32, natural (Sylvester)
 * order, cast back to fp16. signs may be NULL (all +1). x and y are fp16 bit patterns. */
int oracle_hadamard_rotate(const uint16_t *x, int64_t rows, int64_t width, int block,
                           const float *signs, uint16_t *y) {
  if (block <= 0 || (block & (block - 1)) != 0 || width % block != 0) return -1;
  float *tile = (float *)malloc(sizeof(float) * (size_t)block);
  const float scale = 1.0f / sqrtf((float)block);
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t b0 = 0; b0 < width; b0 += block) {
      for (int i = 0; i < block; ++i) {
        tile[i] = half_to_float(x[r * width + b0 + i]) * (signs ? signs[b0 + i] : 1.0f);
      }
      for (int h = 1; h < block; h <<= 1) {
        for (int i = 0; i < block; i += h << 1) {
          for (int j = i; j < i + h; ++j) {
            const float a = tile[j], c = tile[j + h];
            tile[j] = a + c;
            tile[j + h] = a - c;
          }
        }
      }
      for (int i = 0; i < block; ++i) y[r * width + b0 + i] = float_to_half(tile[i] * scale);
    }
  }
  free(tile);
  return 0;
}

/* ---- the product --------------------------------------------------------------------------- */

/* y[m, n] = sum_k x[m, k] * w[n, k], accumulated in double over the exact fp32 weights and the
 * fp16 activations, returned as fp32 (y32) and, rounded once more, as fp16 (y16; may be NULL).
 * Double accumulation makes the oracle's own rounding negligible beside the 2e-3 tolerance. */
static void dot_rows(const float *wrow, const float *xf, int64_t M, int64_t K, int64_t N,
                     int64_t n, float *y32, uint16_t *y16) {
  for (int64_t m = 0; m < M; ++m) {
    const float *xr = xf + m * K;
    double acc = 0.0;
    for (int64_t k = 0; k < K; ++k) acc += (double)xr[k] * (double)wrow[k];
    const float r = (float)acc;
    if (y32) y32[m * N + n] = r;
    if (y16) y16[m * N + n] = float_to_half(r);
  }
}

static float *halves_to_floats(const uint16_t *x, int64_t count) {
  float *xf = (float *)malloc(sizeof(float) * (size_t)count);
  for (int64_t i = 0; i < count; ++i) xf[i] = half_to_float(x[i]);
  return xf;
}

/* Dense fp32 weight [N, K] against fp16 x [M, K]. */
void oracle_matmul(const float *w, const uint16_t *x, int64_t M, int64_t N, int64_t K,
                   float *y32, uint16_t *y16) {
  float *xf = halves_to_floats(x, M * K);
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n) dot_rows(w + n * K, xf, M, K, N, n, y32, y16);
  free(xf);
}

/* GGUF blocks [N][K/256][type size] against fp16 x [M, K]: each row is decoded once, on the fly,
 * and multiplied against every activation row. This is the CPU baseline's shape of the work. */
int oracle_ggml_matmul(int type, const uint8_t *blocks, const uint16_t *x, int64_t M, int64_t N,
                       int64_t K, float *y32, uint16_t *y16) {
  const int ts = oracle_type_size(type);
  if (ts == 0 || K % 256 != 0) return -1;
  const int64_t nb = K / 256;
  float *xf = halves_to_floats(x, M * K);
#pragma omp parallel
  {
    float *row = (float *)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      oracle_dequant(type, blocks + n * nb * ts, nb, row);
      dot_rows(row, xf, M, K, N, n, y32, y16);
    }
    free(row);
  }
  free(xf);
  return 0;
}

/* Affine pack against fp16 x [M, K]; x is used as given (rotate it first for a rotated pack). */
int oracle_affine_matmul(const uint32_t *w, const void *scales, const void *biases,
                         int scale_dtype, int bits, int group_size, const uint16_t *x, int64_t M,
                         int64_t N, int64_t K, float *y32, uint16_t *y16) {
  if (bits < 2 || bits > 8 || K % group_size != 0 || (K * bits) % 32 != 0) return -1;
  const int64_t words = K * bits / 32;
  const int64_t groups = K / group_size;
  float *xf = halves_to_floats(x, M * K);
#pragma omp parallel
  {
    float *row = (float *)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      affine_row(w + n * words, K, bits, group_size, scales, biases, scale_dtype, n * groups, row);
      dot_rows(row, xf, M, K, N, n, y32, y16);
    }
    free(row);
  }
  free(xf);
  return 0;
}

/* ---- dispatch thresholds ------------------------------------------------------------------- */

/* Fewest rows at which the reference routes an affine projection to its verify kernel, by the
 * bytes of the code array. Reference: VerifyMatmul.swift:19-26; pinned by
 * Tests/IshizukiKitTests/VerifyMatmulTests.swift:75-87. */
int oracle_reference_minimum_rows(int64_t bytes) {
  if (bytes >= 100000000) return 2;
  if (bytes >= 10000000) return 3;
  if (bytes >= 5000000) return 4;
  return 6;
}

/* The threads the products above run on; n > 0 sets it (a launcher may have pinned OMP_NUM_THREADS
 * to 1 for its workers, which would make a CPU baseline single-threaded by accident). */
int oracle_set_threads(int n) {
#ifdef _OPENMP
  extern void omp_set_num_threads(int);
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
  return 0;
}

int oracle_threads(void) {
#ifdef _OPENMP
  extern int omp_get_max_threads(void);
  return omp_get_max_threads();
#else
  return 1;
#endif
}
