// The streaming verify-matmul kernel: y[m, n] = sum_k x[m, k] * w[n, k] for 1..16 activation
// rows against a weight that stays in its compressed form.
//
// Shape of the work
//   - A "unit" is 256 consecutive k of one weight row (one GGUF super-block, or the codes and
//     group parameters of 256 k of an affine pack). A "panel" is 16 consecutive output rows.
//   - K is cut into S column ranges; the grid is S groups of Gc persistent CTAs. Within a column
//     range the (panel, unit) pairs are numbered panel-major and dealt to the group's CTAs in
//     equal contiguous runs, so every SM streams the same number of bytes whatever N and K are.
//   - Inside a CTA each consumer warp OWNS units of the column range for the whole kernel: it
//     loads the matching activations once, keeps them in registers in tensor-core fragment
//     order, and then only weights stream past it. A producer warp feeds a ring of panel-sized
//     stages in shared memory with 1-D bulk async copies (one per row segment), completion
//     counted in bytes on an mbarrier.
//   - A panel's partial sums from the warps are added through shared memory by one warp, which
//     writes fp16 outputs directly when the CTA covered the panel's whole K, or parks its fp32
//     partial in a scratch slot; the last CTA to arrive (a counter per panel) adds the slots
//     in a fixed order, so results do not depend on arrival order.
//
// Row segments of formats whose blocks are not multiples of 16 bytes (Q6_K 210, IQ2_XS 74) start
// at 2-byte-aligned addresses. The copy is widened to the enclosing 16-byte-aligned span and the
// consumers index from the remainder; the widened span never leaves the 16-byte chunks that
// hold the segment's first and last bytes.
#pragma once
#include "ishi_ptx.cuh"

namespace ishi {

constexpr int kMaxSrc = 3;
constexpr int kPanelRows = 16;
constexpr int kMaxConsumerWarps = 11;  // plus one producer warp: 384 threads, 168 registers each

struct StreamSrc {
  const uint8_t *base;   // row 0 of this byte stream, 16-byte aligned
  long long row_bytes;   // distance between consecutive rows
  int unit_bytes;        // bytes per row per unit
  int seg_off;           // offset of this stream's segment inside a row slot of a stage
};

struct StreamArgs {
  StreamSrc src[kMaxSrc];
  int nsrc;
  const __half *x;  // [M][K]
  __half *y;
  long long ldy;
  int out_transposed;
  float *scratch;          // [P][S][SL][MT*128]
  unsigned int *counters;  // [P], zero between launches
  int *err;                // set non-zero when a bounded wait gave up
  int M, N, K;
  int units;       // K / 256
  int S;           // column ranges
  int P;           // panels
  int Gc;          // CTAs per column range
  int SL;          // scratch slots per (panel, column range)
  int W;           // consumer warps
  int nstages;
  int row_stride;  // bytes between row slots of a stage
  // format parameters (affine packs)
  int group_size;
  int scale_dtype;
  int rotate_block;  // 0, or a Hadamard block handled while loading the activations
};

// Which CTA of a column group owns quantum q when Q quanta are dealt to Gc CTAs in runs
// [floor(j*Q/Gc), floor((j+1)*Q/Gc)).
__host__ __device__ inline long long cta_of_quantum(long long q, long long Q, long long Gc) {
  return ((q + 1) * Gc - 1) / Q;
}

__host__ __device__ inline int column_begin(int c, int units, int S) {
  return (int)(((long long)c * units) / S);
}

// How many CTAs of column range c contribute to panel p, and (through slot_of) which scratch slot
// CTA j with first quantum q0 takes. When a column range has fewer quanta than CTAs every CTA
// holds at most one quantum, so a panel's contributors are its quanta; otherwise every CTA
// between the owners of the panel's first and last quantum holds part of it.
__host__ __device__ inline int panel_touch(int p, int c, int units, int S, int P, int Gc,
                                           long long *first) {
  const int uc = column_begin(c + 1, units, S) - column_begin(c, units, S);
  const long long Q = (long long)P * uc;
  if (Q < Gc) {
    if (first) *first = -1;
    return uc;
  }
  const long long jf = cta_of_quantum((long long)p * uc, Q, Gc);
  const long long jl = cta_of_quantum((long long)(p + 1) * uc - 1, Q, Gc);
  if (first) *first = jf;
  return (int)(jl - jf + 1);
}

template <class Fmt, int MT, int UW>
__global__ void __launch_bounds__((kMaxConsumerWarps + 1) * 32, 1) stream_kernel(const StreamArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int W = a.W;
  const int nst = a.nstages;
  const int RB = nst + 1;  // reduction buffers: one more than stages, see the finisher below

  // shared memory carve-up
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + nst;
  uint64_t *redbar = empty + nst;
  const uint32_t bars_bytes = (uint32_t)((2 * nst + RB) * 8 + 127) & ~127u;
  const uint32_t red_base = smem_u32(smem) + bars_bytes;
  const uint32_t red_stride = (uint32_t)W * MT * 512u;  // per buffer
  const uint32_t stage_base0 = red_base + (uint32_t)RB * red_stride;
  const uint32_t stage_bytes = (uint32_t)kPanelRows * a.row_stride;
  uint8_t *stage_ptr0 = smem + bars_bytes + (uint32_t)RB * red_stride;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < nst; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], W);
    }
    for (int i = 0; i < RB; ++i) mbar_init(&redbar[i], W);
    mbar_fence_init();
  }
  __syncthreads();
  volatile int *abort_word = &s_abort;

  // this CTA's run of (panel, unit) quanta
  const int c = blockIdx.x / a.Gc;
  const int j = blockIdx.x % a.Gc;
  const int ub0 = column_begin(c, a.units, a.S);
  const int uc = column_begin(c + 1, a.units, a.S) - ub0;
  const long long Q = (long long)a.P * uc;
  const long long q0 = (long long)j * Q / a.Gc;
  const long long q1 = (long long)(j + 1) * Q / a.Gc;
  const int pa = (int)(q0 / uc);
  const int pb = (int)((q1 - 1) / uc);  // inclusive; only meaningful when q1 > q0
  const bool has_work = q1 > q0;

  if (warp == W) {
    // ---------------- producer ----------------
    if (has_work) {
      int it = 0;
      int issued_lo = 0;  // stages [issued_lo, it) may still have copies in flight on abort
      bool ok = true;
      for (int p = pa; p <= pb && ok; ++p, ++it) {
        const int s = it % nst;
        const uint32_t ph = (uint32_t)(it / nst) & 1u;
        if (it >= nst) {
          ok = mbar_wait(&empty[s], ph ^ 1u, abort_word);
          if (!ok) break;
          issued_lo = it - nst + 1;
        }
        const int ua = (p == pa) ? (int)(q0 - (long long)pa * uc) : 0;
        const int ub = (p == pb) ? (int)(q1 - (long long)pb * uc) : uc;
        const long long row = (long long)p * kPanelRows + lane;
        const bool valid = lane < kPanelRows && row < a.N;
        uint32_t bytes[kMaxSrc];
        const uint8_t *from[kMaxSrc];
        uint32_t total = 0;
#pragma unroll
        for (int i = 0; i < kMaxSrc; ++i) {
          bytes[i] = 0;
          from[i] = nullptr;
          if (i < a.nsrc && valid) {
            const uint8_t *g = a.src[i].base + row * a.src[i].row_bytes +
                               (long long)(ub0 + ua) * a.src[i].unit_bytes;
            const uint32_t delta = (uint32_t)((uintptr_t)g & 15u);
            from[i] = g - delta;
            bytes[i] = (delta + (uint32_t)(ub - ua) * a.src[i].unit_bytes + 15u) & ~15u;
            total += bytes[i];
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        if (lane == 0) mbar_arrive_expect_tx(&full[s], total);
        __syncwarp();
        if (valid) {
          uint8_t *dst = stage_ptr0 + (size_t)s * stage_bytes + (size_t)lane * a.row_stride;
#pragma unroll
          for (int i = 0; i < kMaxSrc; ++i) {
            if (i < a.nsrc) bulk_g2s(dst + a.src[i].seg_off, from[i], bytes[i], &full[s]);
          }
        }
      }
      if (!ok) {
        // Gave up: let the copies already issued land before the CTA's shared memory goes away.
        for (int k2 = issued_lo; k2 < it; ++k2) {
          const int s = k2 % nst;
          const uint32_t ph = (uint32_t)(k2 / nst) & 1u;
          for (uint32_t spin = 0; spin < kWaitSpins; ++spin) {
            if (mbar_try_wait(&full[s], ph)) break;
          }
        }
      }
    }
  } else if (warp < W) {
    // ---------------- consumers ----------------
    const int g = lane >> 2;
    const int t = lane & 3;
    typename Fmt::template XFrag<MT, UW> xf;
    Fmt::template load_x<MT, UW>(xf, a, ub0, uc, warp, W, g, t, lane);

    if (has_work) {
      int it = 0;
      bool ok = true;
      for (int p = pa; p <= pb && ok; ++p, ++it) {
        const int s = it % nst;
        const uint32_t ph = (uint32_t)(it / nst) & 1u;
        const int ua = (p == pa) ? (int)(q0 - (long long)pa * uc) : 0;
        const int ub = (p == pb) ? (int)(q1 - (long long)pb * uc) : uc;
        ok = mbar_wait(&full[s], ph, abort_word);
        if (!ok) break;

        float acc[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;

        const uint32_t stage = stage_acquire(stage_base0 + (uint32_t)s * stage_bytes);
        const long long row0 = (long long)p * kPanelRows + g;
#pragma unroll
        for (int q = 0; q < UW; ++q) {
          const int u = warp + q * W;  // unit of the column range owned by this warp
          if (u >= ua && u < ub) {
            Fmt::template unit<MT, UW>(acc, xf, q, a, stage, row0, ub0 + ua, u - ua, g, t);
          }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) values_ready(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);

        // hand the warp's partial tile to the panel's finisher
        const int rb = it % RB;
        const uint32_t red = red_base + (uint32_t)rb * red_stride;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          sts128(red + ((uint32_t)(warp * MT + mt) * 32u + lane) * 16u,
                 make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&redbar[rb]);

        // One warp per panel adds the W partial tiles. It does so before it touches the next
        // panel, and a stage is refilled only after every warp released it, so a buffer written
        // RB = nstages + 1 panels later cannot be overwritten while this warp still reads it.
        if (warp == p % W) {
          ok = mbar_wait(&redbar[rb], (uint32_t)(it / RB) & 1u, abort_word);
          if (!ok) break;
          float sum[MT][4];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            sum[mt][0] = sum[mt][1] = sum[mt][2] = sum[mt][3] = 0.f;
            for (int w2 = 0; w2 < W; ++w2) {
              const float4 v = lds128f(red + ((uint32_t)(w2 * MT + mt) * 32u + lane) * 16u);
              sum[mt][0] += v.x;
              sum[mt][1] += v.y;
              sum[mt][2] += v.z;
              sum[mt][3] += v.w;
            }
          }
          bool write_out = true;
          const bool whole = (a.S == 1) && ua == 0 && ub == uc;
          if (!whole) {
            // park the partial tile, then see whether this CTA is the panel's last contributor
            long long jf;
            panel_touch(p, c, a.units, a.S, a.P, a.Gc, &jf);
            const int slot = jf < 0 ? ua : (int)(j - jf);  // sparse deal: the CTA's single unit
            float *sl = a.scratch + ((((long long)p * a.S + c) * a.SL + slot) * MT) * 128;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              __stcg(reinterpret_cast<float4 *>(sl + mt * 128) + lane,
                     make_float4(sum[mt][0], sum[mt][1], sum[mt][2], sum[mt][3]));
            }
            __threadfence();
            __syncwarp();
            int expected = 0;
            for (int c2 = 0; c2 < a.S; ++c2)
              expected += panel_touch(p, c2, a.units, a.S, a.P, a.Gc, nullptr);
            unsigned int old = 0;
            if (lane == 0) old = atomicAdd(&a.counters[p], 1u);
            old = __shfl_sync(0xffffffffu, old, 0);
            write_out = (int)old == expected - 1;
            if (write_out) {
              __threadfence();
#pragma unroll
              for (int mt = 0; mt < MT; ++mt)
                sum[mt][0] = sum[mt][1] = sum[mt][2] = sum[mt][3] = 0.f;
              for (int c2 = 0; c2 < a.S; ++c2) {
                const int cnt = panel_touch(p, c2, a.units, a.S, a.P, a.Gc, nullptr);
                for (int i = 0; i < cnt; ++i) {
                  const float *s2 = a.scratch + ((((long long)p * a.S + c2) * a.SL + i) * MT) * 128;
#pragma unroll
                  for (int mt = 0; mt < MT; ++mt) {
                    const float4 v = __ldcg(reinterpret_cast<const float4 *>(s2 + mt * 128) + lane);
                    sum[mt][0] += v.x;
                    sum[mt][1] += v.y;
                    sum[mt][2] += v.z;
                    sum[mt][3] += v.w;
                  }
                }
              }
              if (lane == 0) a.counters[p] = 0u;  // ready for the next launch on this stream
            }
          }
          if (write_out) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const long long n = (long long)p * kPanelRows + g + ((i & 2) ? 8 : 0);
                const int m = mt * 8 + 2 * t + (i & 1);
                if (n < a.N && m < a.M) {
                  const __half h = __float2half_rn(sum[mt][i]);
                  if (a.out_transposed) a.y[n * a.ldy + m] = h;
                  else a.y[(long long)m * a.ldy + n] = h;
                }
              }
            }
          }
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && s_abort != 0) atomicExch(a.err, 1);
}

}  // namespace ishi
