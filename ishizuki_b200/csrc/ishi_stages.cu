// RMS norm of the activation rows ahead of a projection (reference: MLXFast.rmsNorm in
// DecoderLayer.callAsFunction, Sources/IshizukiKit/Text/TextModel.swift:151-161): the residual
// stream is fp32 (or fp16), the normalised rows leave in fp16, the width the projections read.
//   y[r][i] = fp16( x[r][i] * rsqrt(mean_i x[r][i]^2 + eps) * w[i] ), arithmetic in fp32.
// Its own launch: the norm needs the whole row's sum of squares before the first value can be
// staged, which a product kernel's CTAs (each reads only its column range, or would all have to read
// the whole fp32 row first) cannot get cheaply. Launched with programmatic stream serialization and
// itself releasing its dependents at once, it overlaps the tail of the launch before and the
// prologue of the product after it.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "ishi_kernels.h"

namespace ishi {

namespace {

template <class T>
__device__ __forceinline__ float to_float(T v) { return (float)v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// one CTA of 256 threads per row; the row stays in registers between the two passes (width <= 256 * kPer)
constexpr int kNormPer = 32;
template <class XT, class WT>
__global__ void __launch_bounds__(256) rms_norm_kernel(const XT *__restrict__ x, const WT *__restrict__ w, long long width, float eps,
                                                       __half *__restrict__ y) {
  __shared__ float part[8];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // x may be the output of the launch before
  const XT *row = x + (long long)blockIdx.x * width;
  float v[kNormPer];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kNormPer; ++j) {
    const long long i = (long long)j * 256 + threadIdx.x;
    v[j] = i < width ? to_float(row[i]) : 0.f;
    ss = fmaf(v[j], v[j], ss);
  }
#pragma unroll
  for (int d = 16; d; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) total += part[i];
  const float r = rsqrtf(total / (float)width + eps);
#pragma unroll
  for (int j = 0; j < kNormPer; ++j) {
    const long long i = (long long)j * 256 + threadIdx.x;
    if (i < width) y[(long long)blockIdx.x * width + i] = __float2half_rn(v[j] * r * to_float(w[i]));
  }
}

template <class XT, class WT>
cudaError_t launch_as(const void *x, const void *w, long long rows, long long width, float eps, __half *y, cudaStream_t st) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)rows);
  cfg.blockDim = dim3(256);
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, rms_norm_kernel<XT, WT>, static_cast<const XT *>(x), static_cast<const WT *>(w), width, eps, y);
}

}  // namespace

long long rms_norm_max_width() { return 256ll * kNormPer; }

// dtypes: 0 fp16, 1 bf16, 2 fp32
cudaError_t launch_rms_norm(const void *x, int x_dtype, const void *w, int w_dtype, long long rows, long long width, float eps,
                            __half *y, cudaStream_t st) {
  if (rows == 0) return cudaSuccess;
  if (x_dtype == 2) {
    if (w_dtype == 2) return launch_as<float, float>(x, w, rows, width, eps, y, st);
    if (w_dtype == 1) return launch_as<float, __nv_bfloat16>(x, w, rows, width, eps, y, st);
    return launch_as<float, __half>(x, w, rows, width, eps, y, st);
  }
  if (x_dtype == 0) {
    if (w_dtype == 2) return launch_as<__half, float>(x, w, rows, width, eps, y, st);
    if (w_dtype == 1) return launch_as<__half, __nv_bfloat16>(x, w, rows, width, eps, y, st);
    return launch_as<__half, __half>(x, w, rows, width, eps, y, st);
  }
  return cudaErrorInvalidValue;
}

}  // namespace ishi
