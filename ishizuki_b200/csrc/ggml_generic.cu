// Kernels that serve every GGML block format through the shared eight-weight decoders: dense
// decode, embedding-row gather, a one-warp-per-output-row product for the formats without a
// streaming kernel of their own, and the arg-max over a row of logits.
#include <cuda_bf16.h>

#include <cmath>
#include <type_traits>

#include "ggml_decode.cuh"
#include "ishi_kernels.h"

namespace ishi {

namespace {

template <typename OT>
__device__ __forceinline__ OT to_out(float v);
template <>
__device__ __forceinline__ float to_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// One warp decodes one block and writes one contiguous run of 256 outputs
// (Sources/IshizukiKit/Core/GGMLKernels.swift:391-401).
template <int TYPE, typename OT>
__global__ void __launch_bounds__(256) ggml_dequantize_kernel(const uint8_t *__restrict__ blocks, long long n_blocks,
                                                              OT *__restrict__ y) {
  constexpr int kBytes = ggml_type_bytes(TYPE);
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long bi = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; bi < n_blocks; bi += warps) {
    float w[8];
    decode8<TYPE>(blocks + bi * kBytes, lane, w);
    OT *out = y + bi * 256 + 8 * lane;
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = to_out<OT>(w[e]);
  }
}

// Rows of a quantized table by id (GGMLKernels.swift:102-138, 404-420): a work item is one block
// of one requested row. Ids outside the table give zeros.
template <int TYPE, typename OT>
__global__ void __launch_bounds__(256) ggml_gather_kernel(const int *__restrict__ ids, long long count,
                                                          const uint8_t *__restrict__ blocks, long long table_rows,
                                                          long long per_row, OT *__restrict__ y) {
  constexpr int kBytes = ggml_type_bytes(TYPE);
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long work = count * per_row;
  for (long long wi = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; wi < work; wi += warps) {
    const long long i = wi / per_row, b = wi - i * per_row;
    const long long row = ids[i];
    float w[8];
    if (row >= 0 && row < table_rows) {
      decode8<TYPE>(blocks + (row * per_row + b) * kBytes, lane, w);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) w[e] = 0.f;
    }
    OT *out = y + wi * 256 + 8 * lane;
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = to_out<OT>(w[e]);
  }
}

// y[m, n] = sum_k x[m, k] * w[n, k]: one warp per output row, every weight decoded once and used
// for all MR activation rows, fp32 accumulation, a warp-shuffle reduction at the end (the shape of
// the reference's ggml_matvec, GGMLKernels.swift:549-565).
template <int TYPE, int MR>
__global__ void __launch_bounds__(256) ggml_rowdot_kernel(const uint8_t *__restrict__ blocks, long long n, long long k,
                                                          const __half *__restrict__ x, int rows, __half *__restrict__ y,
                                                          long long ldy, int transposed) {
  constexpr int kBytes = ggml_type_bytes(TYPE);
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long per_row = k / 256;
  for (long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < n; row += warps) {
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[m] = 0.f;
    const uint8_t *b = blocks + row * per_row * kBytes;
    for (long long bi = 0; bi < per_row; ++bi) {
      float w[8];
      decode8<TYPE>(b + bi * kBytes, lane, w);
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        if (m < rows) {
          const uint4 v = __ldg(reinterpret_cast<const uint4 *>(x + (long long)m * k + bi * 256 + 8 * lane));
          const uint32_t p[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&p[e]));
            acc[m] = fmaf(w[2 * e], f.x, acc[m]);
            acc[m] = fmaf(w[2 * e + 1], f.y, acc[m]);
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
#pragma unroll
      for (int d = 16; d >= 1; d >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], d);
      if (lane == 0 && m < rows) {
        if (transposed) y[row * ldy + m] = __float2half_rn(acc[m]);
        else y[(long long)m * ldy + row] = __float2half_rn(acc[m]);
      }
    }
  }
}

// Index of the largest of n fp16 logits per row, the lowest index among equals (MLX argMax as the
// greedy verify uses it, Sources/IshizukiKit/Generate/SpeculativeGeneration.swift:173-177). NaN
// never wins. A row is cut into chunks, one CTA each (grid: chunks x rows): 16-byte loads where the
// row allows, the chunk's best (value, index) goes to `parts`, and the CTA that counts itself last
// for its row reduces the row's parts. Value first, then the lower index: the result does not
// depend on the order in which the CTAs finish. `counters` (one per row) are zero between launches.
struct ArgPart {
  float v;
  int i;
};
__device__ __forceinline__ bool arg_better(float v, int i, float bv, int bi) {
  return i >= 0 && (bi < 0 || v > bv || (v == bv && i < bi));
}
__device__ __forceinline__ void arg_take(float v, int i, float &best, int &at) {
  if (v > best || (at < 0 && v == best)) best = v, at = i;  // indices come in ascending order per thread
}
__global__ void __launch_bounds__(256) argmax_rows_kernel(const __half *__restrict__ y, long long n, long long ldy, int chunk,
                                                          ArgPart *__restrict__ parts, unsigned *__restrict__ counters,
                                                          int *__restrict__ out) {
  __shared__ float s_val[8];
  __shared__ int s_idx[8];
  __shared__ bool s_last;
  const int r = blockIdx.y, c = blockIdx.x, nchunks = gridDim.x;
  const __half *row = y + (long long)r * ldy;
  const long long lo = (long long)c * chunk, hi = lo + chunk < n ? lo + chunk : n;
  float best = -INFINITY;
  int at = -1;
  long long i = lo + (long long)threadIdx.x * 8;
  if ((reinterpret_cast<uintptr_t>(row + lo) & 15u) == 0) {
    for (; i + 8 <= hi; i += 256 * 8) {
      const uint4 q = *reinterpret_cast<const uint4 *>(row + i);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[e]));
        arg_take(f.x, (int)i + 2 * e, best, at);
        arg_take(f.y, (int)i + 2 * e + 1, best, at);
      }
    }
  }
  // what the 16-byte loads left: a misaligned chunk, the last few values
  for (; i < hi; i += 256 * 8)
    for (long long k = i; k < hi && k < i + 8; ++k) arg_take(__half2float(row[k]), (int)k, best, at);
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, d);
    const int oi = __shfl_xor_sync(0xffffffffu, at, d);
    if (arg_better(ov, oi, best, at)) best = ov, at = oi;
  }
  if ((threadIdx.x & 31) == 0) s_val[threadIdx.x >> 5] = best, s_idx[threadIdx.x >> 5] = at;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (arg_better(s_val[w], s_idx[w], best, at)) best = s_val[w], at = s_idx[w];
    parts[(long long)r * nchunks + c] = ArgPart{best, at};
    __threadfence();
    const unsigned before = atomicAdd(counters + r, 1u);
    s_last = before == (unsigned)nchunks - 1;
  }
  __syncthreads();
  if (!s_last || threadIdx.x >= 32) return;
  __threadfence();
  best = -INFINITY, at = -1;
  for (int k = threadIdx.x; k < nchunks; k += 32) {
    const ArgPart *pt = parts + (long long)r * nchunks + k;
    const float pv = __ldcg(&pt->v);  // written by other CTAs of this launch: from L2
    const int pi = __ldcg(&pt->i);
    if (arg_better(pv, pi, best, at)) best = pv, at = pi;
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, d);
    const int oi = __shfl_xor_sync(0xffffffffu, at, d);
    if (arg_better(ov, oi, best, at)) best = ov, at = oi;
  }
  if (threadIdx.x == 0) {
    out[r] = at < 0 ? 0 : at;
    counters[r] = 0;  // for the next launch on this stream
  }
}

template <class F>
cudaError_t with_type(int type, F &&f) {
  switch (type) {
    case 10: f(std::integral_constant<int, 10>()); break;
    case 12: f(std::integral_constant<int, 12>()); break;
    case 14: f(std::integral_constant<int, 14>()); break;
    case 16: f(std::integral_constant<int, 16>()); break;
    case 17: f(std::integral_constant<int, 17>()); break;
    case 18: f(std::integral_constant<int, 18>()); break;
    case 19: f(std::integral_constant<int, 19>()); break;
    case 21: f(std::integral_constant<int, 21>()); break;
    case 22: f(std::integral_constant<int, 22>()); break;
    case 23: f(std::integral_constant<int, 23>()); break;
    case 29: f(std::integral_constant<int, 29>()); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace

int ggml_type_size(int type) { return ggml_type_bytes(type); }

cudaError_t launch_ggml_dequantize(int type, const uint8_t *blocks, long long n_blocks, void *out, int out_dtype, int sm_count,
                                   cudaStream_t st) {
  const long long want = (n_blocks * 32 + 255) / 256;
  const int grid = (int)(want < (long long)sm_count * 32 ? want : (long long)sm_count * 32);
  return with_type(type, [&](auto t) {
    constexpr int T = decltype(t)::value;
    if (out_dtype == 0) ggml_dequantize_kernel<T, __half><<<grid, 256, 0, st>>>(blocks, n_blocks, static_cast<__half *>(out));
    else if (out_dtype == 1)
      ggml_dequantize_kernel<T, __nv_bfloat16><<<grid, 256, 0, st>>>(blocks, n_blocks, static_cast<__nv_bfloat16 *>(out));
    else ggml_dequantize_kernel<T, float><<<grid, 256, 0, st>>>(blocks, n_blocks, static_cast<float *>(out));
  });
}

cudaError_t launch_ggml_gather(int type, const int *ids, long long count, const uint8_t *blocks, long long table_rows,
                               long long k, void *out, int out_dtype, int sm_count, cudaStream_t st) {
  const long long per_row = k / 256;
  const long long want = (count * per_row * 32 + 255) / 256;
  const int grid = (int)(want < (long long)sm_count * 32 ? want : (long long)sm_count * 32);
  return with_type(type, [&](auto t) {
    constexpr int T = decltype(t)::value;
    if (out_dtype == 0)
      ggml_gather_kernel<T, __half><<<grid, 256, 0, st>>>(ids, count, blocks, table_rows, per_row, static_cast<__half *>(out));
    else if (out_dtype == 1)
      ggml_gather_kernel<T, __nv_bfloat16>
          <<<grid, 256, 0, st>>>(ids, count, blocks, table_rows, per_row, static_cast<__nv_bfloat16 *>(out));
    else ggml_gather_kernel<T, float><<<grid, 256, 0, st>>>(ids, count, blocks, table_rows, per_row, static_cast<float *>(out));
  });
}

cudaError_t launch_ggml_rowdot(int type, const uint8_t *blocks, long long n, long long k, const __half *x, int rows, __half *y,
                               long long ldy, int transposed, int sm_count, cudaStream_t st) {
  const long long want = (n * 32 + 255) / 256;
  const int grid = (int)(want < (long long)sm_count * 16 ? want : (long long)sm_count * 16);
  return with_type(type, [&](auto t) {
    constexpr int T = decltype(t)::value;
    if (rows <= 4) ggml_rowdot_kernel<T, 4><<<grid, 256, 0, st>>>(blocks, n, k, x, rows, y, ldy, transposed);
    else if (rows <= 8) ggml_rowdot_kernel<T, 8><<<grid, 256, 0, st>>>(blocks, n, k, x, rows, y, ldy, transposed);
    else ggml_rowdot_kernel<T, 16><<<grid, 256, 0, st>>>(blocks, n, k, x, rows, y, ldy, transposed);
  });
}

// scratch: ishi::argmax_scratch_bytes() bytes, zero before the first launch
size_t argmax_scratch_bytes() { return (size_t)16 * 1024 * sizeof(ArgPart) + 16 * sizeof(unsigned); }

cudaError_t launch_argmax_rows(const __half *y, int rows, long long n, long long ldy, int *out, void *scratch, cudaStream_t st) {
  if (rows < 1 || rows > 16 || n < 1 || n > 0x7fffffffll) return cudaErrorInvalidValue;
  long long chunk = 8192;
  while ((n + chunk - 1) / chunk > 1024) chunk *= 2;
  const int nchunks = (int)((n + chunk - 1) / chunk);
  ArgPart *parts = static_cast<ArgPart *>(scratch);
  unsigned *counters = reinterpret_cast<unsigned *>(parts + 16 * 1024);
  argmax_rows_kernel<<<dim3(nchunks, rows), 256, 0, st>>>(y, n, ldy, (int)chunk, parts, counters, out);
  return cudaGetLastError();
}

}  // namespace ishi
