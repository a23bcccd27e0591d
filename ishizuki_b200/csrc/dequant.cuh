// The dense decoder of affine packs and the stand-alone Hadamard rotation. They define "the
// decoded weight values" and "the rotated activations" bit for bit (the MLX affine formula, the
// reference's fused rotation kernel), so every product below is written with explicit
// single-rounding intrinsics in the reference's order of operations and nothing here may be
// compiled with fast-math. (The GGML block decoders are in ggml_decode.cuh.)
#pragma once
#include <cuda_bf16.h>

#include "iq2xs_tables.h"
#include "ishi_ptx.cuh"

namespace ishi {

static __constant__ uint16_t c_iq2xs_codes[512] = {ISHI_IQ2XS_CODES_LIST};

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
