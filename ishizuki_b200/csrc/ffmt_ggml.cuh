// The eight other GGML block types (Q2_K, IQ2_XXS, IQ2_S, IQ3_XXS, IQ3_S, IQ1_S, IQ1_M, IQ4_XS) on the
// warp-level kernel through the dense decoder, the comparison path beside their own fragment
// decoders (ISHI_DENSE_DECODER=1 at projection create): no bit tricks here, a lane decodes the
// sixteen weights of a sub-block with decode8 (ggml_decode.cuh, the same code that defines the
// decoded weight values) and rounds them to fp16 pairs for the MMA. Reference: the block bodies at
// Sources/IshizukiKit/Core/GGMLKernels.swift:568-582,630-761 and GGMLDequant.swift:125-150,222-428.
//
// Rounding the decoded weight to fp16 costs at most 2^-11 of each weight; against the fp16
// rounding of the output itself and the tolerance of the product (2e-3 of the largest output)
// that is small, and the tests hold these formats to the same tolerance as the others.
//
// Fragment mapping as for IQ2_XS (m16n8k16; lane g = lane / 4, t = lane % 4 holds weight rows g
// and g + 8): a lane owns the sub-blocks of sixteen weights 4 j + t, j = 0..3, of both rows; the
// eight registers of a sub-block feed four k-steps (slots (2t, 2t + 1) = weights 4m, 4m + 1,
// slots (2t + 8, 2t + 9) = weights 4m + 2, 4m + 3), so the activations are used as they lie in
// memory: 32 contiguous bytes of x per lane and sub-block.
//
// Tile (16 rows x 256 k): the sixteen blocks as they are, row after row. Activations of a unit in
// shared memory: eight rows of 256 fp16 as they lie in x, umax * 512 + 16 bytes apart.
#pragma once
#include "ggml_decode.cuh"
#include "ishi_fragstream.cuh"

namespace ishi {

template <int TYPE>
struct FragGGML {
  static constexpr int kBlock = ggml_type_bytes(TYPE);
  static_assert(kBlock > 0, "a GGML type with a decoder");
  static constexpr int kTileBytes = 16 * kBlock;
  static constexpr int kXBytes = 8 * 512;  // per unit: eight rows of 512 bytes
  static constexpr int kExtraBytes = 8 * 16;  // the rows' 16-byte skews
  static constexpr bool kRowMode = false;     // one activation row runs through the MMA path as well

  static __device__ __forceinline__ uint8_t tile_byte(const FragSrc &s, long long p, int u, int b) {
    const long long row = p * kFragRows + b / kBlock;
    if (row >= s.N) return 0;  // a block of zeros decodes to zeros in every one of these formats
    long long local;
    const int seg = frag_segment(s, row, &local);
    return s.w[seg][local * s.w_row_bytes + (long long)u * kBlock + b % kBlock];
  }
  static __device__ __forceinline__ uint16_t tile_halfword(const FragSrc &s, long long p, int u, int hw) {
    return (uint16_t)(tile_byte(s, p, u, 2 * hw) | ((uint32_t)tile_byte(s, p, u, 2 * hw + 1) << 8));
  }

  static __device__ __forceinline__ uint32_t row_stride(const FragArgs &a) { return (uint32_t)a.umax * 512u + 16u; }

  // nothing to set up ahead of the dependency wait
  static __device__ __forceinline__ void before_wait(const FragArgs &, uint32_t) {}

  // Activations of the CTA's column range as they lie in x (rows past M as zeros). A warp task is
  // (unit, activation row): lane l loads and stores k = 8l .. 8l + 7. after_loads() runs once,
  // when the first batch of loads is in flight. GGML blocks have no input rotation.
  template <class F>
  static __device__ __forceinline__ void stage_x(const FragArgs &a, uint32_t xfrag, int ub0, int uc, F &&after_loads) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const uint32_t R = row_stride(a);
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
        sts128u(xfrag + (uint32_t)(i & 7) * R + (uint32_t)(i >> 3) * 512u + (uint32_t)lane * 16u, v[e]);
      }
    }
  }

  // eight decoded weights as four A registers (fp16 pairs)
  static __device__ __forceinline__ void pack(uint32_t (&r)[4], const float (&w)[8]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h = __floats2half2_rn(w[2 * i], w[2 * i + 1]);
      r[i] = *reinterpret_cast<const uint32_t *>(&h);
    }
  }

  // One tile against the activations of its unit; acc is the warp's C fragment.
  template <int MODE>
  static __device__ __forceinline__ void unit(float (&acc)[4], const FragArgs &a, uint32_t tile, uint32_t xbase, int uq,
                                              int g, int t, int lane) {
    (void)lane;
    const uint32_t R = row_stride(a);
    const uint32_t xrow = xbase + (uint32_t)g * R + (uint32_t)uq * 512u + (uint32_t)t * 32u;
    const uint8_t *blk0 = static_cast<const uint8_t *>(__cvta_shared_to_generic(tile + (uint32_t)g * kBlock));
    const uint8_t *blk1 = static_cast<const uint8_t *>(__cvta_shared_to_generic(tile + (uint32_t)(g + 8) * kBlock));
#pragma unroll 1
    for (int j = 0; j < 4; ++j) {
      const int sb = 4 * j + t;
      float w[8];
      uint32_t lo0[4], hi0[4], lo1[4], hi1[4];
      decode8<TYPE>(blk0, 2 * sb, w);
      pack(lo0, w);
      decode8<TYPE>(blk0, 2 * sb + 1, w);
      pack(hi0, w);
      decode8<TYPE>(blk1, 2 * sb, w);
      pack(lo1, w);
      decode8<TYPE>(blk1, 2 * sb + 1, w);
      pack(hi1, w);
      const uint4 b0 = lds128(xrow + (uint32_t)j * 128u), b1 = lds128(xrow + (uint32_t)j * 128u + 16u);
      mma16816(acc, lo0[0], lo1[0], lo0[1], lo1[1], b0.x, b0.y);
      mma16816(acc, lo0[2], lo1[2], lo0[3], lo1[3], b0.z, b0.w);
      mma16816(acc, hi0[0], hi1[0], hi0[1], hi1[1], b1.x, b1.y);
      mma16816(acc, hi0[2], hi1[2], hi0[3], hi1[3], b1.z, b1.w);
    }
  }
};

}  // namespace ishi
