// Dense decoders: GGUF blocks or affine packs to a dense array. These define "the decoded
// weight values": they must equal ggml's to_float (reference restatement:
// Sources/IshizukiKit/Core/GGMLDequant.swift) and the MLX affine formula bit for bit, so every
// product below is written with explicit single-rounding intrinsics in the reference's order
// of operations and nothing here may be compiled with fast-math.
//
// One warp decodes one block, lane L the eight weights 8L .. 8L+7, as the reference's Metal
// decoder does (Sources/IshizukiKit/Core/GGMLKernels.swift:391-401): a warp then writes one
// contiguous 1 KB (fp32) run per block.
#pragma once
#include <cuda_bf16.h>

#include "iq2xs_tables.h"
#include "ishi_ptx.cuh"

namespace ishi {

static __constant__ uint16_t c_iq2xs_codes[512] = {ISHI_IQ2XS_CODES_LIST};

template <typename OT>
__device__ __forceinline__ OT to_out(float v);
template <>
__device__ __forceinline__ float to_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float rd_half(const uint8_t *p) {
  return half_bits_to_float((uint32_t)p[0] | ((uint32_t)p[1] << 8));
}

// GGMLDequant.swift:187-220
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

// GGMLDequant.swift:154-185
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

// GGMLDequant.swift:264-285; the sign byte of index i is i with bit 7 = parity(i)
// (Sources/IshizukiKit/Core/GGMLTables.swift:15-24 lists exactly these values).
__device__ __forceinline__ void decode8_iq2xs(const uint8_t *b, int lane, float (&w)[8]) {
  const int ib = lane >> 2, l = lane & 3;
  const uint32_t sbyte = b[66 + ib];
  const uint32_t s = l < 2 ? (sbyte & 0xfu) : (sbyte >> 4);
  const float db = __fmul_rn(__fmul_rn(rd_half(b), 0.5f + (float)s), 0.25f);
  const uint32_t q = (uint32_t)b[2 + 2 * lane] | ((uint32_t)b[3 + 2 * lane] << 8);
  const uint32_t codes = c_iq2xs_codes[q & 511u];
  const uint32_t s7 = q >> 9;
  const uint32_t signs = s7 | ((__popc(s7) & 1u) << 7);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const uint32_t c = (codes >> (2 * e)) & 3u;
    const float gv = c == 0 ? (float)ISHI_IQ2XS_VALUE0 : (c == 1 ? (float)ISHI_IQ2XS_VALUE1 : (float)ISHI_IQ2XS_VALUE2);
    w[e] = __fmul_rn(__fmul_rn(db, gv), ((signs >> e) & 1u) ? -1.0f : 1.0f);
  }
}

template <int TYPE, typename OT>
__global__ void __launch_bounds__(256) ggml_dequantize_kernel(const uint8_t *__restrict__ blocks,
                                                              long long n_blocks, OT *__restrict__ y) {
  constexpr int kBytes = TYPE == 12 ? 144 : (TYPE == 14 ? 210 : 74);
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long bi = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; bi < n_blocks; bi += warps) {
    const uint8_t *b = blocks + bi * kBytes;
    float w[8];
    if (TYPE == 12) decode8_q4k(b, lane, w);
    else if (TYPE == 14) decode8_q6k(b, lane, w);
    else decode8_iq2xs(b, lane, w);
    OT *out = y + bi * 256 + 8 * lane;
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = to_out<OT>(w[e]);
  }
}

// w = float(code) * scale + bias (Sources/IshizukiKit/Core/VerifyMatmul.swift:282-287); code i of
// a row sits at bit i * bits of the row's little-endian word stream.
__device__ __forceinline__ float load_scale(const void *p, long long i, int dtype) {
  if (dtype == 0) return __half2float(((const __half *)p)[i]);
  if (dtype == 1) return __bfloat162float(((const __nv_bfloat16 *)p)[i]);
  return ((const float *)p)[i];
}

static __global__ void __launch_bounds__(256) affine_dequantize_kernel(const uint32_t *__restrict__ w,
                                                                const void *__restrict__ scales,
                                                                const void *__restrict__ biases,
                                                                int scale_dtype, int group_size, int bits,
                                                                long long n, long long k, float *__restrict__ y) {
  const long long total = n * k;
  const long long words = k * bits / 32;
  const uint32_t mask = (1u << bits) - 1u;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / k, col = i - row * k;
    const long long bit = col * bits;
    const uint32_t *rw = w + row * words;
    const int off = (int)(bit & 31);
    uint32_t v = rw[bit >> 5] >> off;
    if (off + bits > 32) v |= rw[(bit >> 5) + 1] << (32 - off);
    const long long gi = row * (k / group_size) + col / group_size;
    const float s = load_scale(scales, gi, scale_dtype), b = load_scale(biases, gi, scale_dtype);
    y[i] = __fadd_rn(__fmul_rn((float)(v & mask), s), b);
  }
}

// xr = WHT_block(x * signs) / sqrt(block), fp32 inside, fp16 out; natural (Sylvester) order.
// One CTA per (row, block); the radix-2 stages run in shared memory exactly in the order of the
// reference's fused kernel (Sources/IshizukiKit/Core/FusedHadamard.swift:54-78) so the fp32
// roundings agree.
static __global__ void __launch_bounds__(256) hadamard_rotate_kernel(const __half *__restrict__ x, long long width,
                                                              int block, const float *__restrict__ signs,
                                                              __half *__restrict__ y) {
  extern __shared__ float tile[];
  const long long blocks_per_row = width / block;
  const long long row = blockIdx.x / blocks_per_row;
  const long long bir = blockIdx.x % blocks_per_row;
  const long long base = row * width + bir * block;
  for (int i = threadIdx.x; i < block; i += blockDim.x) {
    const float s = signs ? signs[bir * block + i] : 1.0f;
    tile[i] = __fmul_rn(__half2float(x[base + i]), s);
  }
  __syncthreads();
  for (int h = 1; h < block; h <<= 1) {
    for (int b = threadIdx.x; b < block / 2; b += blockDim.x) {
      const int j = (b / h) * (h << 1) + (b % h);
      const float a = tile[j], c = tile[j + h];
      tile[j] = __fadd_rn(a, c);
      tile[j + h] = __fsub_rn(a, c);
    }
    __syncthreads();
  }
  const float scale = 1.0f / sqrtf((float)block);
  for (int i = threadIdx.x; i < block; i += blockDim.x) y[base + i] = __float2half_rn(__fmul_rn(tile[i], scale));
}

}  // namespace ishi
