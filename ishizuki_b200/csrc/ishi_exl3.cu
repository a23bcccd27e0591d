// EXL3 trellis-coded weights: decode, rotations and the few-row product that decodes inside the
// matrix multiply (reference: Sources/IshizukiKit/Core/EXL3.swift).
//
// W [k, n] is stored as 16 x 16 tiles, tile (tk, tn) at ((tk * n / 16) + tn) * ring / 32 32-bit
// words; a tile is a ring of 256 * bits bits (half-integer rates: 128 * (2 * whole + 1)), each word
// counted from its top bit. Weight p of a tile is a function (one of three procedural codebooks,
// EXL3.swift:171-182) of the 16 ring bits that end where p's own code ends (EXL3.swift:184-214).
// Weight p = 8 * lane + i lies at row (lane % 4) * 2 + {0, 1, 8, 9}[i % 4], column
// lane / 4 + 8 * (i / 4) (EXL3.swift:286-290): with the weight's output dimension n on the M side of
// mma.sync m16n8k16 (A[n][k]) that is exactly lane's A fragment of one k-step,
//   a0 = (v0, v1), a1 = (v4, v5), a2 = (v2, v3), a3 = (v6, v7),
// so a tile is decoded straight into tensor-core operands and never written anywhere.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "ishi_kernels.h"
#include "ishi_ptx.cuh"

namespace ishi {

namespace {

// ring bits of a tile
__host__ __device__ constexpr int exl3_ring(int whole, bool half) { return half ? 128 * (2 * whole + 1) : 256 * whole; }

// bit of the ring where weight p's code ends
template <int KA, bool HK>
__device__ __forceinline__ uint32_t exl3_end(uint32_t p) {
  return HK ? (p >> 1) * (2 * KA + 1) + KA + (p & 1) * (KA + 1) : (p + 1) * KA;
}
// the same for weight 8 * lane + i, relative to the start of lane's first 16-bit window
template <int KA, bool HK>
__host__ __device__ constexpr uint32_t exl3_rel(uint32_t i) {
  return HK ? (i >> 1) * (2 * KA + 1) + (i & 1) * (KA + 1) + 16 : i * KA + 16;
}

// Two weights of 16-bit states s0, s1 as one fp16 pair (s0 in the low half).
// Codebooks 3INST and MCG (mul1 == false): x = s * mult + add; the two halves of
// (x & 0x8fff8fff) ^ 0x3b603b60 are fp16 numbers whose fp16 sum is the weight.
// Codebook MUL1: the byte sum of s * 0x83DCD12D as the mantissa of an fp16 in [1024, 2048), then one
// fused multiply-add in fp16.
template <bool MUL1>
__device__ __forceinline__ uint32_t exl3_pair(uint32_t s0, uint32_t s1, uint32_t mult, uint32_t add) {
  if (MUL1) {
    // the byte sums through the four-way byte dot product with 0x6400 as its addend; the second
    // weight's sum, moved to the upper half, is the addend of the first
    const uint32_t m1 = __dp4a(s1 * 0x83DCD12Du, 0x01010101u, 0x6400u);
    const uint32_t h = __dp4a(s0 * 0x83DCD12Du, 0x01010101u, (m1 << 16) + 0x6400u);
    const uint32_t m = 0x1eee1eeeu, b = 0xc931c931u;
    const __half2 r = __hfma2(*reinterpret_cast<const __half2 *>(&h), *reinterpret_cast<const __half2 *>(&m),
                              *reinterpret_cast<const __half2 *>(&b));
    return *reinterpret_cast<const uint32_t *>(&r);
  }
  const uint32_t x0 = ((s0 * mult + add) & 0x8fff8fffu) ^ 0x3b603b60u;
  const uint32_t x1 = ((s1 * mult + add) & 0x8fff8fffu) ^ 0x3b603b60u;
  const uint32_t lo = prmt(x0, x1, 0x5410u), hi = prmt(x0, x1, 0x7632u);  // (x0.lo, x1.lo), (x0.hi, x1.hi)
  const __half2 r = __hadd2(*reinterpret_cast<const __half2 *>(&lo), *reinterpret_cast<const __half2 *>(&hi));
  return *reinterpret_cast<const uint32_t *>(&r);
}

// Which three consecutive ring words (with wrap-around) hold lane's eight 16-bit windows, and the
// bit of the first word where the first window starts. The same for every tile of a rate.
template <int KA, bool HK>
struct Exl3Lane {
  uint32_t j0, j1, j2, sh;
  __device__ __forceinline__ explicit Exl3Lane(int lane) {
    constexpr uint32_t kRing = exl3_ring(KA, HK), kWords = kRing / 32;
    const uint32_t lo = exl3_end<KA, HK>((uint32_t)lane * 8u) + kRing - 16u;  // first bit of the first window
    const uint32_t i0 = lo >> 5;
    sh = lo & 31u;
    j0 = i0 >= kWords ? i0 - kWords : i0;
    j1 = j0 + 1 >= kWords ? j0 + 1 - kWords : j0 + 1;
    j2 = j1 + 1 >= kWords ? j1 + 1 - kWords : j1 + 1;
  }
};

// lane's eight weights of one tile, from its three ring words, as four fp16 pairs (v0 v1 | v2 v3 | v4 v5 | v6 v7)
template <int KA, bool HK, bool MUL1>
__device__ __forceinline__ void exl3_decode8(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t sh, uint32_t mult, uint32_t add,
                                             uint32_t (&v)[4]) {
  // 96 ring bits from the window's first bit on: b0 (top) b1 b2
  const uint32_t b0 = __funnelshift_l(w1, w0, sh), b1 = __funnelshift_l(w2, w1, sh), b2 = w2 << sh;
  uint32_t s[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t r = exl3_rel<KA, HK>((uint32_t)i);  // the state is bits r - 16 ... r - 1 of the 96
    uint32_t x;
    if (r <= 32) x = b0 >> (32 - r);
    else if (r < 64) x = __funnelshift_l(b1, b0, r - 32);  // bits r - 32 ... r - 1
    else if (r == 64) x = b1;
    else x = __funnelshift_l(b2, b1, r - 64);
    s[i] = x & 0xffffu;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = exl3_pair<MUL1>(s[2 * i], s[2 * i + 1], mult, add);
}

// ---- dequantize: one warp per tile ----------------------------------------------------------------
template <int KA, bool HK, bool MUL1, class OT>
__global__ void __launch_bounds__(256) exl3_dequantize_kernel(const uint32_t *__restrict__ trellis, int tiles_k, int tiles_n,
                                                              uint32_t mult, uint32_t add, OT *__restrict__ w) {
  constexpr uint32_t kWords = exl3_ring(KA, HK) / 32;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)tiles_k * tiles_n;
  const long long N = (long long)tiles_n * 16;
  for (long long tile = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); tile < total; tile += (long long)gridDim.x * 8) {
    uint32_t v[4];
    const Exl3Lane<KA, HK> at(lane);
    const uint32_t *words = trellis + tile * kWords;
    exl3_decode8<KA, HK, MUL1>(__ldg(words + at.j0), __ldg(words + at.j1), __ldg(words + at.j2), at.sh, mult, add, v);
    const long long row = (tile / tiles_n) * 16 + (lane & 3) * 2, col = (tile % tiles_n) * 16 + (lane >> 2);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __half2 pair = *reinterpret_cast<const __half2 *>(&v[i >> 1]);
      const float f = (i & 1) ? __high2float(pair) : __low2float(pair);
      const int dr = (i & 1) + ((i & 2) ? 8 : 0), dc = (i & 4) ? 8 : 0;
      w[(row + dr) * N + col + dc] = (OT)f;
    }
  }
}

// ---- the product: y [rows][n] fp32 = x [rows][k] fp16 . W --------------------------------------------
// One CTA per C adjacent tile columns (16 C outputs), its sixteen warps split the k tiles. For a k
// tile a warp reads the matching 16 inputs of up to eight rows once (B: lane (g, t) reads
// x[g][16 tk + 2t, 2t + 1] and [.. + 8, + 9]), decodes the C tiles, which lie one after the other in
// memory, each into its A fragment, and multiplies. The words of two k tiles are requested before
// the first is decoded. The warps' partial 16 x 8 tiles are added through shared memory in a
// fixed order.
constexpr int kExl3Warps = 16;
template <int KA, bool HK, bool MUL1, int C>
__global__ void __launch_bounds__(kExl3Warps * 32) exl3_matvec_kernel(const uint32_t *__restrict__ trellis, int tiles_k, int tiles_n,
                                                                      uint32_t mult, uint32_t add, const __half *__restrict__ x,
                                                                      int rows, long long K, float *__restrict__ y) {
  constexpr uint32_t kWords = exl3_ring(KA, HK) / 32;
  __shared__ float red[kExl3Warps][C][32][4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int tn0 = blockIdx.x * C;
  float acc[C][4];
#pragma unroll
  for (int c = 0; c < C; ++c) acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;
  const Exl3Lane<KA, HK> at(lane);
  const uint32_t *column = trellis + (long long)tn0 * kWords;
  const long long tile_stride = (long long)tiles_n * kWords;
  const uint32_t *xr = reinterpret_cast<const uint32_t *>(x + (long long)g * K) + t;  // pairs of inputs
  const bool live = g < rows;
  constexpr int kUnroll = 2;
  for (int tk0 = warp; tk0 < tiles_k; tk0 += kExl3Warps * kUnroll) {
    uint32_t w[kUnroll][C][3], b[kUnroll][2];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int tk = tk0 + kExl3Warps * u;
      if (tk < tiles_k) {
        const uint32_t *tiles = column + tk * tile_stride;
#pragma unroll
        for (int c = 0; c < C; ++c) {
          w[u][c][0] = __ldg(tiles + c * kWords + at.j0);
          w[u][c][1] = __ldg(tiles + c * kWords + at.j1);
          w[u][c][2] = __ldg(tiles + c * kWords + at.j2);
        }
        b[u][0] = live ? __ldg(xr + tk * 8) : 0u;
        b[u][1] = live ? __ldg(xr + tk * 8 + 4) : 0u;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (tk0 + kExl3Warps * u < tiles_k) {
#pragma unroll
        for (int c = 0; c < C; ++c) {
          uint32_t v[4];
          exl3_decode8<KA, HK, MUL1>(w[u][c][0], w[u][c][1], w[u][c][2], at.sh, mult, add, v);
          mma16816(acc[c], v[0], v[2], v[1], v[3], b[u][0], b[u][1]);
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < C; ++c)
#pragma unroll
    for (int i = 0; i < 4; ++i) red[warp][c][lane][i] = acc[c][i];
  __syncthreads();
  for (int e = threadIdx.x; e < C * 128; e += kExl3Warps * 32) {
    const int c = e >> 7, l = (e >> 2) & 31, i = e & 3;  // accumulator i of lane l, column c
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kExl3Warps; ++w) s += red[w][c][l][i];
    // lane (g, t): c0, c1 = output g, rows 2t, 2t + 1; c2, c3 = output g + 8
    const int out = (l >> 2) + ((i & 2) ? 8 : 0), m = 2 * (l & 3) + (i & 1);
    if (m < rows) y[(long long)m * tiles_n * 16 + (tn0 + c) * 16 + out] = s;
  }
}

// ---- rotation: block Hadamard of 128 with a scale vector before or after (EXL3.swift:219-262) -------
template <class IT, class OT>
__global__ void __launch_bounds__(256) exl3_rotate_kernel(const IT *__restrict__ x, const __half *__restrict__ s, long long blocks,
                                                          int blocks_per_row, int pre, OT *__restrict__ y) {
  const int lane = threadIdx.x & 31;
  for (long long block = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); block < blocks; block += (long long)gridDim.x * 8) {
    const long long base = block * 128 + lane * 4;
    const long long col = (block % blocks_per_row) * 128 + lane * 4;
    float v[4], sc[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = (float)x[base + i];
      sc[i] = __half2float(s[col + i]);
      if (pre) v[i] = __fmul_rn(v[i], sc[i]);
    }
    const float a0 = __fadd_rn(v[0], v[1]), a1 = __fsub_rn(v[0], v[1]), a2 = __fadd_rn(v[2], v[3]), a3 = __fsub_rn(v[2], v[3]);
    v[0] = __fadd_rn(a0, a2), v[2] = __fsub_rn(a0, a2), v[1] = __fadd_rn(a1, a3), v[3] = __fsub_rn(a1, a3);
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float p = __shfl_xor_sync(0xffffffffu, v[i], m);
        v[i] = (lane & m) ? __fsub_rn(p, v[i]) : __fadd_rn(v[i], p);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = __fmul_rn(v[i], 0.08838834764831845f);
      if (!pre) v[i] = __fmul_rn(v[i], sc[i]);
      y[base + i] = (OT)v[i];
    }
  }
}

template <int KA, bool HK, bool MUL1>
cudaError_t dequantize_as(const uint32_t *trellis, int tiles_k, int tiles_n, uint32_t mult, uint32_t add, void *out, int out_dtype,
                          int sm_count, cudaStream_t st) {
  const long long total = (long long)tiles_k * tiles_n;
  const int grid = (int)((total + 7) / 8 < (long long)sm_count * 8 ? (total + 7) / 8 : (long long)sm_count * 8);
  if (out_dtype == 2)
    exl3_dequantize_kernel<KA, HK, MUL1, float><<<grid, 256, 0, st>>>(trellis, tiles_k, tiles_n, mult, add, static_cast<float *>(out));
  else
    exl3_dequantize_kernel<KA, HK, MUL1, __half><<<grid, 256, 0, st>>>(trellis, tiles_k, tiles_n, mult, add, static_cast<__half *>(out));
  return cudaGetLastError();
}

// C tile columns per CTA: as many (up to four) as still leave one and a half CTAs per SM
template <int KA, bool HK, bool MUL1>
cudaError_t matvec_as(const uint32_t *trellis, int tiles_k, int tiles_n, uint32_t mult, uint32_t add, const __half *x, int rows,
                      float *y, int sm_count, cudaStream_t st) {
  const long long K = (long long)tiles_k * 16;
  const int threads = kExl3Warps * 32;
  if (tiles_n % 4 == 0 && tiles_n / 4 >= sm_count * 3 / 2)
    exl3_matvec_kernel<KA, HK, MUL1, 4><<<tiles_n / 4, threads, 0, st>>>(trellis, tiles_k, tiles_n, mult, add, x, rows, K, y);
  else if (tiles_n % 2 == 0 && tiles_n / 2 >= sm_count * 3 / 2)
    exl3_matvec_kernel<KA, HK, MUL1, 2><<<tiles_n / 2, threads, 0, st>>>(trellis, tiles_k, tiles_n, mult, add, x, rows, K, y);
  else
    exl3_matvec_kernel<KA, HK, MUL1, 1><<<tiles_n, threads, 0, st>>>(trellis, tiles_k, tiles_n, mult, add, x, rows, K, y);
  return cudaGetLastError();
}

// rate (16-bit words per tile = 16 * bits) and codebook to the template arguments
template <class F>
cudaError_t by_rate(int words16, int codebook, F &&f) {
  const bool half = (words16 & 15) != 0;
  const int whole = words16 >> 4;
  if (codebook < 0 || codebook > 2 || (words16 & 7) || whole < 1 || whole > 8 || (half && (whole > 3 || codebook != 2)))
    return cudaErrorInvalidValue;
#define ISHI_EXL3_CASE(KA)                                                          \
  case KA:                                                                          \
    return codebook == 2 ? f(std::integral_constant<int, KA>(), std::false_type(), std::true_type()) \
                         : f(std::integral_constant<int, KA>(), std::false_type(), std::false_type());
  if (!half) {
    switch (whole) {
      ISHI_EXL3_CASE(1)
      ISHI_EXL3_CASE(2)
      ISHI_EXL3_CASE(3)
      ISHI_EXL3_CASE(4)
      ISHI_EXL3_CASE(5)
      ISHI_EXL3_CASE(6)
      ISHI_EXL3_CASE(7)
      ISHI_EXL3_CASE(8)
    }
  }
#undef ISHI_EXL3_CASE
  switch (whole) {
    case 1: return f(std::integral_constant<int, 1>(), std::true_type(), std::true_type());
    case 2: return f(std::integral_constant<int, 2>(), std::true_type(), std::true_type());
    case 3: return f(std::integral_constant<int, 3>(), std::true_type(), std::true_type());
  }
  return cudaErrorInvalidValue;
}

// multiplier and addend of the two codebooks that share a kernel
void codebook_constants(int codebook, uint32_t *mult, uint32_t *add) {
  *mult = codebook == 1 ? 0xCBAC1FEDu : 89226354u;
  *add = codebook == 1 ? 0u : 64248484u;
}

}  // namespace

bool exl3_rate_supported(int words16, int codebook) {
  const bool half = (words16 & 15) != 0;
  const int whole = words16 >> 4;
  return codebook >= 0 && codebook <= 2 && !(words16 & 7) && whole >= 1 && whole <= 8 && !(half && (whole > 3 || codebook != 2));
}

cudaError_t launch_exl3_dequantize(const int16_t *trellis, int tiles_k, int tiles_n, int words16, int codebook, void *out,
                                   int out_dtype, int sm_count, cudaStream_t st) {
  uint32_t mult, add;
  codebook_constants(codebook, &mult, &add);
  return by_rate(words16, codebook, [&](auto ka, auto hk, auto mul1) {
    return dequantize_as<decltype(ka)::value, decltype(hk)::value, decltype(mul1)::value>(
        reinterpret_cast<const uint32_t *>(trellis), tiles_k, tiles_n, mult, add, out, out_dtype, sm_count, st);
  });
}

cudaError_t launch_exl3_matvec(const int16_t *trellis, int tiles_k, int tiles_n, int words16, int codebook, const __half *x,
                               int rows, float *y, int sm_count, cudaStream_t st) {
  uint32_t mult, add;
  codebook_constants(codebook, &mult, &add);
  return by_rate(words16, codebook, [&](auto ka, auto hk, auto mul1) {
    return matvec_as<decltype(ka)::value, decltype(hk)::value, decltype(mul1)::value>(reinterpret_cast<const uint32_t *>(trellis),
                                                                                      tiles_k, tiles_n, mult, add, x, rows, y, sm_count, st);
  });
}

cudaError_t launch_exl3_rotate(const void *x, int x_dtype, long long rows, long long width, const __half *scales, int before,
                               void *y, int y_dtype, int sm_count, cudaStream_t st) {
  const long long blocks = rows * (width / 128);
  if (blocks == 0) return cudaSuccess;
  const int grid = (int)((blocks + 7) / 8 < (long long)sm_count * 8 ? (blocks + 7) / 8 : (long long)sm_count * 8);
  const int bpr = (int)(width / 128);
  if (x_dtype == 0 && y_dtype == 0)
    exl3_rotate_kernel<__half, __half><<<grid, 256, 0, st>>>(static_cast<const __half *>(x), scales, blocks, bpr, before, static_cast<__half *>(y));
  else if (x_dtype == 0 && y_dtype == 2)
    exl3_rotate_kernel<__half, float><<<grid, 256, 0, st>>>(static_cast<const __half *>(x), scales, blocks, bpr, before, static_cast<float *>(y));
  else if (x_dtype == 2 && y_dtype == 0)
    exl3_rotate_kernel<float, __half><<<grid, 256, 0, st>>>(static_cast<const float *>(x), scales, blocks, bpr, before, static_cast<__half *>(y));
  else if (x_dtype == 2 && y_dtype == 2)
    exl3_rotate_kernel<float, float><<<grid, 256, 0, st>>>(static_cast<const float *>(x), scales, blocks, bpr, before, static_cast<float *>(y));
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace ishi
