// The warp-level verify-matmul kernel: y[m, n] = sum_k x[m, k] * w[n, k] for 1..8 activation rows
// on mma.sync (m16n8k16, weights on the M side, activation rows on the N side), with a CUDA-core
// variant for a single row.
//
// Why not tcgen05 here: one tcgen05.mma of 128 weight rows x 16 k costs about 100 cycles of the
// SM's tensor pipe whatever N is (measured for N = 16 ... 128), which caps a few-row product at
// ~20 weights per clock and SM; eight activation rows fill an m16n8k16 fragment exactly, and the
// warp-level instruction sustains several times that. The tcgen05 kernel stays for the formats
// that have no fragment decoder yet.
//
// Layout. The weight is re-tiled once, when the projection is created, into fragment order: a
// tile is 16 output rows x 256 k (one unit), stored as [16-byte piece][lane] so that every
// warp-wide 128-bit access is one contiguous 512-byte run, followed by a small per-row section
// (block scales). Lane (g = lane / 4, t = lane % 4) owns weight rows g and g + 8 of the tile and,
// in every k-step, the four k positions the format's decoder assigns to t. Same bytes as the raw
// weight, different order.
//
// Work. K is cut into S column ranges, the grid into S groups of Gc persistent CTAs; (panel,
// unit) pairs of a column range are dealt to its CTAs in equal contiguous runs. Inside a CTA the
// activations of the column range are staged once into shared memory in fragment order, and warp
// w takes the units u = w, w + W, ... of every panel. Each warp streams its tiles through a
// private ring in shared memory with cp.async (16 bytes per lane), so there is no producer warp
// and no cross-warp wait on the data path; the warps meet once per panel (a CTA barrier) to add
// their partial tiles. A panel whose units are spread over several CTAs goes through fp32
// scratch slots and an arrival counter; the last contributor adds the slots in slot order. That
// commit is deferred to the end of the CTA so its latency is paid once, not per panel.
#pragma once
#include "ishi_stream.cuh"

namespace ishi {

constexpr int kFragRows = 16;
constexpr int kFragMaxWarps = 16;
constexpr int kFragRing = 4;  // tiles per warp-private ring: three in flight while one is decoded

struct FragArgs {
  const uint8_t *tiles;  // [P][units][tile_bytes]
  int tile_bytes;        // 16 rows x bytes of one unit
  int ring_stride;       // tile_bytes rounded up to 128
  const __half *x;
  __half *y;
  long long ldy;
  int out_transposed;
  float *scratch;          // [P][S][SL][128]
  unsigned int *counters;  // [P]
  int M, N, K;
  int units, S, P, Gc, SL, W;
  int umax;                // most units in a column range
  int group_size, scale_dtype;
};

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
  asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}

__host__ __device__ inline int frag_column_begin(int c, int units, int S) { return (int)(((long long)c * units) / S); }

// contributors to panel p: per column range as panel_touch(); slot order is column-major
__host__ __device__ inline int frag_touch(int p, int c, int units, int S, int P, int Gc, long long *first) {
  const int uc = frag_column_begin(c + 1, units, S) - frag_column_begin(c, units, S);
  return panel_touch(p, uc, P, Gc, first);
}

// MODE 0: tensor-core (rows 1..8); MODE 1: CUDA-core FMA for a single row.
template <class Fmt, int MODE>
__global__ void __launch_bounds__(kFragMaxWarps * 32, 1) frag_kernel(const FragArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int W = a.W;

  // shared memory: activations in fragment order, partial tiles, one ring per warp
  const uint32_t xfrag = smem_u32(smem);                                   // [umax][Fmt::kXBytes]
  const uint32_t red = xfrag + (uint32_t)a.umax * Fmt::kXBytes;            // [2][W][32 lanes][16 B]
  const uint32_t ring = red + 2u * (uint32_t)W * 512u + (uint32_t)warp * kFragRing * (uint32_t)a.ring_stride;

  const int c = blockIdx.x / a.Gc;
  const int j = blockIdx.x % a.Gc;
  const int ub0 = frag_column_begin(c, a.units, a.S);
  const int uc = frag_column_begin(c + 1, a.units, a.S) - ub0;
  const long long Q = (long long)a.P * uc;
  const long long q0 = (long long)j * Q / a.Gc;
  const long long q1 = (long long)(j + 1) * Q / a.Gc;
  const bool has_work = q1 > q0;
  const int pa = has_work ? (int)(q0 / uc) : 0;
  const int pb = has_work ? (int)((q1 - 1) / uc) : -1;  // inclusive
  const int npanels = pb - pa + 1;
  const int ua_first = (int)(q0 - (long long)pa * uc);
  const int ub_last = (int)(q1 - (long long)pb * uc);
  const int per = (uc - 1 - warp + W) / W;  // units of a full panel this warp owns (u = warp + i * W < uc)
  const int perw = per > 0 ? per : 1;

  // This warp's tile sequence: panel pa + pi, unit warp + qi * W for qi < perw, panel after panel;
  // a tile is present when its unit lies inside the CTA's part of that panel. Every warp walks the
  // same panels. Two cursors run over the sequence: the fetch cursor kFragRing - 1 tiles ahead of
  // the compute cursor. No division on this path.
  auto present = [&](int pi, int qi) -> bool {
    const int u = warp + qi * W;
    return pi < npanels && u < uc && (pi != 0 || u >= ua_first) && (pi != npanels - 1 || u < ub_last);
  };
  int f_pi = 0, f_qi = 0;
  uint32_t f_slot = ring;
  const uint32_t ring_end = ring + kFragRing * (uint32_t)a.ring_stride;
  const uint8_t *f_src = a.tiles + ((long long)pa * a.units + ub0 + warp) * (long long)a.tile_bytes;
  const long long step_unit = (long long)W * a.tile_bytes;
  const long long step_panel = (long long)(a.units - perw * W) * a.tile_bytes;
  auto fetch = [&]() {
    if (present(f_pi, f_qi)) {
      for (int o = lane * 16; o < a.tile_bytes; o += 512) cp_async16(f_slot + o, f_src + o);
    }
    cp_async_commit();  // one group per slot, present or not, so the wait below counts slots
    f_src += step_unit;
    if (++f_qi == perw) {
      f_qi = 0;
      ++f_pi;
      f_src += step_panel;
    }
    f_slot += (uint32_t)a.ring_stride;
    if (f_slot == ring_end) f_slot = ring;
  };

  if (has_work) {
#pragma unroll
    for (int i = 0; i < kFragRing - 1; ++i) fetch();
  }

  // activations of the column range into fragment order (all warps), while the first tiles fly
  Fmt::stage_x(a, xfrag, ub0, uc);
  __syncthreads();
  // shared-memory loads are plain asm the compiler may move; tie their addresses to the waits
  const uint32_t xf = stage_acquire(xfrag) + (uint32_t)warp * Fmt::kXBytes;

  if (has_work) {
    uint32_t c_slot = ring;
    for (int pi = 0; pi < npanels; ++pi) {
      const int p = pa + pi;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t xq = xf;
      for (int qi = 0; qi < perw; ++qi) {
        fetch();
        cp_async_wait<kFragRing - 1>();  // this slot has landed (the younger groups may still be in flight)
        __syncwarp();
        if (present(pi, qi)) {
          Fmt::template unit<MODE>(acc, a, stage_acquire(c_slot), xq, g, t, lane);
          values_ready(acc[0], acc[1], acc[2], acc[3]);
        }
        __syncwarp();  // every lane is done reading the slot before it is refilled
        xq += (uint32_t)W * Fmt::kXBytes;
        c_slot += (uint32_t)a.ring_stride;
        if (c_slot == ring_end) c_slot = ring;
      }
      if (MODE == 1) {
        // single activation row: each lane holds partial dot products of rows g (acc[0]) and
        // g + 8 (acc[2]) over its own k positions; add across the four lanes of a row
        acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 1);
        acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 2);
        acc[2] += __shfl_xor_sync(0xffffffffu, acc[2], 1);
        acc[2] += __shfl_xor_sync(0xffffffffu, acc[2], 2);
        if (t != 0) acc[0] = acc[2] = 0.f;  // one copy per row enters the sum below (column m = 0)
        acc[1] = acc[3] = 0.f;
      }
      // add the warps' partial tiles: one warp per panel
      const uint32_t rb = red + (uint32_t)(pi & 1) * (uint32_t)W * 512u;
      sts128(rb + ((uint32_t)warp * 32u + lane) * 16u, make_float4(acc[0], acc[1], acc[2], acc[3]));
      __syncthreads();
      if (warp == pi % W) {
        const uint32_t rbs = stage_acquire(rb);
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
        for (int w2 = 0; w2 < W; ++w2) {
          const float4 v = lds128f(rbs + ((uint32_t)w2 * 32u + lane) * 16u);
          sum[0] += v.x;
          sum[1] += v.y;
          sum[2] += v.z;
          sum[3] += v.w;
        }
        const int ua = (p == pa) ? ua_first : 0, ub = (p == pb) ? ub_last : uc;
        const bool whole = a.S == 1 && ua == 0 && ub == uc;
        if (whole) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const long long n = (long long)p * kFragRows + g + ((e & 2) ? 8 : 0);
            const int m = 2 * t + (e & 1);
            if (n < a.N && m < a.M) {
              const __half h = __float2half_rn(sum[e]);
              if (a.out_transposed) a.y[n * a.ldy + m] = h;
              else a.y[(long long)m * a.ldy + n] = h;
            }
          }
        } else {
          // park the partial tile; it is committed after the loop
          long long jf;
          frag_touch(p, c, a.units, a.S, a.P, a.Gc, &jf);
          const int slot = jf < 0 ? ua : (int)(j - jf);
          float *sl = a.scratch + (((long long)p * a.S + c) * a.SL + slot) * 128;
          __stcg(reinterpret_cast<float4 *>(sl) + lane, make_float4(sum[0], sum[1], sum[2], sum[3]));
        }
      }
    }

    // deferred commit of the panels this warp finished that were shared with other CTAs
    __threadfence();
    for (int pi = warp; pi < npanels; pi += W) {
      const int p = pa + pi;
      const int ua = (p == pa) ? ua_first : 0, ub = (p == pb) ? ub_last : uc;
      if (a.S == 1 && ua == 0 && ub == uc) continue;
      int expected = 0;
      for (int c2 = 0; c2 < a.S; ++c2) expected += frag_touch(p, c2, a.units, a.S, a.P, a.Gc, nullptr);
      unsigned int old = 0;
      if (lane == 0) old = atomicAdd(&a.counters[p], 1u);
      old = __shfl_sync(0xffffffffu, old, 0);
      if ((int)old != expected - 1) continue;
      __threadfence();
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
      for (int c2 = 0; c2 < a.S; ++c2) {
        const int cnt = frag_touch(p, c2, a.units, a.S, a.P, a.Gc, nullptr);
        for (int i = 0; i < cnt; ++i) {
          const float *s2 = a.scratch + (((long long)p * a.S + c2) * a.SL + i) * 128;
          const float4 v = __ldcg(reinterpret_cast<const float4 *>(s2) + lane);
          sum[0] += v.x;
          sum[1] += v.y;
          sum[2] += v.z;
          sum[3] += v.w;
        }
      }
      if (lane == 0) a.counters[p] = 0u;  // ready for the next launch on this stream
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const long long n = (long long)p * kFragRows + g + ((e & 2) ? 8 : 0);
        const int m = 2 * t + (e & 1);
        if (n < a.N && m < a.M) {
          const __half h = __float2half_rn(sum[e]);
          if (a.out_transposed) a.y[n * a.ldy + m] = h;
          else a.y[(long long)m * a.ldy + n] = h;
        }
      }
    }
  }
  cp_async_wait<0>();
}

// One-time re-tiling into fragment order: Fmt::tile_halfword says which 2 bytes of the source
// land at halfword hw of tile (p, u). Rows past N read as zero.
struct FragSrc {
  const uint8_t *w, *scales, *biases;  // GGUF blocks, or an affine pack's three arrays
  long long w_row_bytes, s_row_bytes;  // distance between rows
  long long N;
  int group_size, scale_bytes;
};

template <class Fmt>
__global__ void __launch_bounds__(256) prepare_frag_kernel(const FragSrc src, int units, int tile_bytes,
                                                           uint8_t *__restrict__ dst) {
  const long long P = (src.N + kFragRows - 1) / kFragRows;
  const int halfwords = tile_bytes / 2;
  const long long total = P * units * halfwords;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int hw = (int)(i % halfwords);
    const long long pu = i / halfwords;
    const int u = (int)(pu % units);
    const long long p = pu / units;
    reinterpret_cast<uint16_t *>(dst + pu * (long long)tile_bytes)[hw] = Fmt::tile_halfword(src, p, u, hw);
  }
}

}  // namespace ishi
