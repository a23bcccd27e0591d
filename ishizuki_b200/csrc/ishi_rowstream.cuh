// The tcgen05 verify-matmul kernel: y[m, n] = sum_k x[m, k] * w[n, k] for 1..8 activation rows,
// the weight streamed in its compressed form and decoded once, one weight row per thread.
//
// Roles inside a CTA (224 threads, two CTAs per SM):
//   warps 0-3  decode: thread r owns output row r of the current 128-row panel. It reads its
//              row's bytes from the stage in shared memory, turns codes into exact fp16 values in
//              registers and writes them straight into tensor memory (tcgen05.st) as the A operand;
//              later it reads its row of the accumulator back (tcgen05.ld), applies the row's
//              fp32 scales and keeps the running sums in registers.
//   warp 4     producer: one bulk async copy per stage into a ring of stages. The weight is read
//              from a "tiled" copy made once when the projection is created: for every (panel,
//              unit) the 128 row blocks sit back to back, so the units a stage needs are one
//              contiguous, 16-byte aligned run whatever the block size (144, 210, 74 bytes ...).
//              Same bytes, same compression; only the order in memory changes. (One copy per
//              weight-row segment, the layout-preserving alternative, is limited by the copy
//              engine's per-instruction cost at 128 small copies a stage.)
//   warp 5     activations: loads the x slice of a stage, stores it in the tensor core's
//              K-major core-matrix layout (in the k order the decoders emit), and the per-group
//              sums of x that the minimum / bias term needs.
//   warp 6     one thread issues tcgen05.mma (M = 128 weight rows, N = 16, K = 16 per
//              instruction; A from tensor memory, B = x from shared memory) and commits.
//
// A "step" is 128 consecutive k of the panel: one A buffer of 64 tensor-memory columns, split
// into G accumulation groups that each get their own 16-column accumulator, because each group
// has its own per-row scale. The decode threads run one step ahead of the tensor core: while
// the MMAs of step H run they apply the scales of step H-1 and decode step H+1.
//
// Work is dealt as in the warp-level kernel: (panel, unit) pairs numbered panel-major and cut
// into equal contiguous runs, one per CTA; a panel shared by several CTAs is combined through
// fp32 scratch slots and a per-(panel, warp) arrival counter, the last arrival adding the slots
// in a fixed order.
//
// Every wait is bounded (see mbar_wait); a CTA that gives up still waits for its copies, frees
// its tensor memory and raises the error word.
#pragma once
#include "ishi_stream.cuh"

namespace ishi {

constexpr int kRowPanel = 128;
constexpr int kRowThreads = 224;
constexpr int kTmemCols = 256;
// tensor-memory column map
constexpr uint32_t kColA0 = 0, kColA1 = 64, kColD = 128, kColAmin = 192, kColDmin = 208;

struct RowArgs {
  const uint8_t *tiles;  // [P][units][tile_bytes]: see prepare_tiles_kernel
  int tile_bytes;        // 128 rows x bytes of one unit, all byte streams of the format
  int sec_off[4];        // offset of each section (128 rows x field bytes) inside a tile
  int sec_bytes[4];      // bytes per row of each section
  const __half *x;
  __half *y;
  long long ldy;
  int out_transposed;
  float *scratch;          // [P][SL][8][128]
  unsigned int *counters;  // [P][4]
  int *err;
  int M, N, K;
  int units;       // K / 256
  int P;           // panels of 128 rows
  int SL;          // scratch slots per panel
  int kc;          // units per stage
  int nstages;
  int x_off;       // offset of the activation chunk inside a stage
  int bmin_off;    // offset of the group-sum MMA operand inside a stage (formats with a minimum term)
  int xs_off;      // offset of the fp32 group sums of x inside a stage (affine packs: bias term)
  int stage_bytes;
  int group_size, scale_dtype, bits;
};

// ---- tcgen05 wrappers ---------------------------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&d)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]), "=f"(d[4]), "=f"(d[5]), "=f"(d[6]), "=f"(d[7])
               : "r"(taddr)
               : "memory");
}

__device__ __forceinline__ void tmem_ld4(uint32_t taddr, float (&d)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld2(uint32_t taddr, float (&d)[2]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0,%1}, [%2];" : "=f"(d[0]), "=f"(d[1]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld1(uint32_t taddr, float (&d)[1]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=f"(d[0]) : "r"(taddr) : "memory");
}
// the first MC accumulator columns of this thread's row
template <int MC>
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, float (&d)[MC]);
template <>
__device__ __forceinline__ void tmem_ldn<8>(uint32_t taddr, float (&d)[8]) { tmem_ld8(taddr, d); }
template <>
__device__ __forceinline__ void tmem_ldn<4>(uint32_t taddr, float (&d)[4]) { tmem_ld4(taddr, d); }
template <>
__device__ __forceinline__ void tmem_ldn<2>(uint32_t taddr, float (&d)[2]) { tmem_ld2(taddr, d); }
template <>
__device__ __forceinline__ void tmem_ldn<1>(uint32_t taddr, float (&d)[1]) { tmem_ld1(taddr, d); }

// D[tmem_d] (+)= A[tmem_a] * B[desc]; M = 128, N = 16, K = 16, fp16 in, fp32 out. The accumulate
// flag is almost always a compile-time constant at the call site, so the two cases are separate
// instructions with a constant predicate instead of a computed one.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  if (accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 1, 1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 1, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc)
        : "memory");
  }
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// K-major, no swizzle: 8 x 16-byte core matrices, 128 bytes apart along K; the second group of
// eight B rows sits sbo bytes further (0 aliases it onto the first group: rows 8..15 of the
// accumulator then repeat rows 0..7 and are never read).
__device__ __forceinline__ uint64_t make_bdesc(uint32_t smem_addr, uint32_t sbo_bytes) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(128u >> 4) << 16) |
         ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46);
}
constexpr uint32_t kIdescF16 = (1u << 4) | ((uint32_t)(16 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

// ---- the walk over a CTA's run of (panel, unit) quanta, identical in every role --------------------

struct RowWalk {
  long long q, q1;
  int units, kc;
  __device__ __forceinline__ RowWalk(const RowArgs &a) : units(a.units), kc(a.kc) {
    const long long Q = (long long)a.P * a.units;
    q = (long long)blockIdx.x * Q / gridDim.x;
    q1 = (long long)(blockIdx.x + 1) * Q / gridDim.x;
  }
  // One stage: panel p, units [u0, u0 + nu) of it. Returns false when the run is exhausted.
  __device__ __forceinline__ bool next(int &p, int &u0, int &nu, bool &last_of_panel) {
    if (q >= q1) return false;
    p = (int)(q / units);
    u0 = (int)(q - (long long)p * units);
    long long end = (long long)(p + 1) * units;
    if (end > q1) end = q1;
    long long take = end - q;
    if (take > kc) take = kc;
    nu = (int)take;
    q += take;
    last_of_panel = (q == end);
    return true;
  }
};

// MC: accumulator columns read back and kept per row (the activation rows rounded up to 1, 2, 4
// or 8); the MMAs always compute the full tile.
template <class Fmt, int MC>
__global__ void __launch_bounds__(kRowThreads, 2) rowstream_kernel(const RowArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_abort;
  __shared__ uint32_t s_tmem;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nst = a.nstages;

  uint64_t *full = reinterpret_cast<uint64_t *>(smem);  // producer + activation warp + bytes
  uint64_t *empty = full + nst;                         // 4 decode warps + the tensor core's commit
  uint64_t *a_ready = empty + nst;                      // 4 decode warps: A stored, D of the step before read
  uint64_t *mma_done = a_ready + 1;                     // tensor core's commit for a step
  const uint32_t bars_bytes = 128;
  uint8_t *table = smem + bars_bytes;  // format's lookup table, if it has one
  uint8_t *stage0 = table + Fmt::kTableBytes;
  const uint32_t stage0_u32 = smem_u32(stage0);

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < nst; ++i) {
      mbar_init(&full[i], 2);
      mbar_init(&empty[i], 5);
    }
    mbar_init(a_ready, 4);
    mbar_init(mma_done, 1);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(&s_tmem, kTmemCols);
  Fmt::build_table(table, threadIdx.x, blockDim.x);
  // the second 16-byte core matrix of every group-sum operand stays zero for the whole kernel
  for (int i = threadIdx.x; Fmt::kHasMin && i < nst * a.kc * 2 * 64; i += blockDim.x) {
    const int st = i / (a.kc * 2 * 64), rem = i % (a.kc * 2 * 64);
    reinterpret_cast<uint32_t *>(stage0 + (size_t)st * a.stage_bytes + a.bmin_off)[rem] = 0u;
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  volatile int *abort_word = &s_abort;
  const uint32_t tmem = s_tmem;

  RowWalk walk(a);
  int p, u0, nu;
  bool last;

  if (warp == 4) {
    // ---------------- producer: one copy per stage ----------------
    int it = 0, issued_lo = 0;
    bool ok = true;
    while (ok && walk.next(p, u0, nu, last)) {
      const int s = it % nst;
      const uint32_t ph = (uint32_t)(it / nst) & 1u;
      if (it >= nst) {
        ok = mbar_wait(&empty[s], ph ^ 1u, abort_word);
        if (!ok) break;
        issued_lo = it - nst + 1;
      }
      if (lane == 0) {
        const uint32_t bytes = (uint32_t)nu * (uint32_t)a.tile_bytes;
        mbar_arrive_expect_tx(&full[s], bytes);
        bulk_g2s(stage0 + (size_t)s * a.stage_bytes,
                 a.tiles + ((long long)p * a.units + u0) * (long long)a.tile_bytes, bytes, &full[s]);
      }
      __syncwarp();
      ++it;
    }
    if (!ok) {
      for (int k2 = issued_lo; k2 < it; ++k2) {
        const int s = k2 % nst;
        const uint32_t ph = (uint32_t)(k2 / nst) & 1u;
        for (uint32_t spin = 0; spin < kWaitSpins; ++spin)
          if (mbar_try_wait(&full[s], ph)) break;
      }
    }
  } else if (warp == 5) {
    // ---------------- activations: x slice -> core matrices, group sums ----------------
    int it = 0;
    bool ok = true;
    while (ok && walk.next(p, u0, nu, last)) {
      const int s = it % nst;
      const uint32_t ph = (uint32_t)(it / nst) & 1u;
      typename Fmt::XRegs xv;
      Fmt::load_x(a, u0, nu, lane, xv);  // in flight while the stage drains
      if (it >= nst) ok = mbar_wait(&empty[s], ph ^ 1u, abort_word);
      if (!ok) break;
      Fmt::store_x(a, stage0_u32 + (uint32_t)s * a.stage_bytes, nu, lane, xv);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full[s]);
      ++it;
    }
  } else if (warp == 6) {
    // ---------------- tensor core issue ----------------
    // every operand of the MMA instruction has to sit in a uniform register; the tensor-memory
    // base was read from shared memory, so a warp reduction tells the compiler it is uniform
    const uint32_t tmem_u = __reduce_or_sync(0xffffffffu, tmem);
    int it = 0;
    uint32_t H = 0;
    bool ok = true;
    while (ok && walk.next(p, u0, nu, last)) {
      const int s = it % nst;
      const uint32_t ph = (uint32_t)(it / nst) & 1u;
      ok = mbar_wait(&full[s], ph, abort_word);
      if (!ok) break;
      const uint32_t xbase = stage0_u32 + (uint32_t)s * a.stage_bytes + a.x_off;
      const uint32_t mbase = stage0_u32 + (uint32_t)s * a.stage_bytes + a.bmin_off;
      for (int hs = 0; hs < 2 * nu && ok; ++hs, ++H) {
        ok = mbar_wait(a_ready, H & 1u, abort_word);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t acol = tmem_u + ((H & 1u) ? kColA1 : kColA0);
          Fmt::issue_step(a, tmem_u, acol, make_bdesc(xbase + (uint32_t)hs * 2048u, 0u),
                          make_bdesc(mbase + (uint32_t)hs * 256u, 0u), hs & 1);
          umma_commit(mma_done);
          if (hs == 2 * nu - 1) umma_commit(&empty[s]);
        }
        __syncwarp();
      }
      ++it;
    }
  } else {
    // ---------------- decode: one weight row per thread ----------------
    const int r = threadIdx.x;  // row inside the panel; also this thread's tensor-memory lane
    const uint32_t tlane = tmem + ((uint32_t)(warp * 32) << 16);
    typename Fmt::RowState rs;
    Fmt::init_state(rs, smem_u32(table));
    float acc[MC];
#pragma unroll
    for (int m = 0; m < MC; ++m) acc[m] = 0.f;
    int it = 0;
    uint32_t H = 0;
    bool pending = false;  // accumulators of step H-1 not yet read back
    bool ok = true;
    int first_unit_of_panel = -1;
    int release_s = -1;  // a stage is handed back only after the sums of its last step were used
    while (ok && walk.next(p, u0, nu, last)) {
      const int s = it % nst;
      const uint32_t ph = (uint32_t)(it / nst) & 1u;
      if (first_unit_of_panel < 0) first_unit_of_panel = u0;
      ok = mbar_wait(&full[s], ph, abort_word);
      if (!ok) break;
      const uint32_t stage = stage_acquire(stage0_u32 + (uint32_t)s * a.stage_bytes);
      const long long row = (long long)p * kRowPanel + r;
      for (int ul = 0; ul < nu && ok; ++ul) {
        const uint32_t ra = stage + (uint32_t)ul * (uint32_t)a.tile_bytes;  // this unit's tile
        Fmt::begin_unit(rs, a, ra, r);
#pragma unroll
        for (int hh = 0; hh < 2; ++hh, ++H) {
          Fmt::decode_step(rs, a, ra, r, hh, tlane + ((H & 1u) ? kColA1 : kColA0));
          if (pending) {
            ok = mbar_wait(mma_done, (H - 1u) & 1u, abort_word);
            if (!ok) break;
            tc_fence_after();
            Fmt::template consume_step<MC>(rs, a, acc, tlane);
            if (release_s >= 0) {
              __syncwarp();
              if (lane == 0) mbar_arrive(&empty[release_s]);
              release_s = -1;
            }
          }
          Fmt::store_min(rs, hh, tlane);
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(a_ready);
          Fmt::advance(rs, hh, stage + a.xs_off + (uint32_t)(2 * ul + hh) * 128u);
          pending = true;
        }
      }
      if (!ok) break;
      release_s = s;
      ++it;

      if (last) {
        // drain the tensor core for this panel, then write it out
        ok = mbar_wait(mma_done, (H - 1u) & 1u, abort_word);
        if (!ok) break;
        tc_fence_after();
        Fmt::template consume_step<MC>(rs, a, acc, tlane);
        pending = false;
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[release_s]);
        release_s = -1;

        const bool whole = first_unit_of_panel == 0 && u0 + nu == a.units;
        bool write_out = true;
        if (!whole) {
          long long jf;
          const int cnt = panel_touch(p, a.units, a.P, (int)gridDim.x, &jf);
          const int slot = jf < 0 ? first_unit_of_panel : (int)(blockIdx.x - jf);
          float *sl = a.scratch + (((long long)p * a.SL + slot) * 8) * kRowPanel + r;
#pragma unroll
          for (int m = 0; m < MC; ++m) __stcg(sl + m * kRowPanel, acc[m]);
          __threadfence();
          __syncwarp();
          unsigned int old = 0;
          if (lane == 0) old = atomicAdd(&a.counters[p * 4 + warp], 1u);
          old = __shfl_sync(0xffffffffu, old, 0);
          write_out = (int)old == cnt - 1;
          if (write_out) {
            __threadfence();
#pragma unroll
            for (int m = 0; m < MC; ++m) acc[m] = 0.f;
            for (int i = 0; i < cnt; ++i) {
              const float *s2 = a.scratch + (((long long)p * a.SL + i) * 8) * kRowPanel + r;
#pragma unroll
              for (int m = 0; m < MC; ++m) acc[m] += __ldcg(s2 + m * kRowPanel);
            }
            if (lane == 0) a.counters[p * 4 + warp] = 0u;
          }
        }
        if (write_out && row < a.N) {
#pragma unroll
          for (int m = 0; m < MC; ++m) {
            if (m < a.M) {
              const __half h = __float2half_rn(acc[m]);
              if (a.out_transposed) a.y[row * a.ldy + m] = h;
              else a.y[(long long)m * a.ldy + row] = h;
            }
          }
        }
#pragma unroll
        for (int m = 0; m < MC; ++m) acc[m] = 0.f;
        first_unit_of_panel = -1;
      }
    }
    if (ok && release_s >= 0) {
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[release_s]);
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
  if (threadIdx.x == 0 && s_abort != 0) atomicExch(a.err, 1);
}

// One-time re-tiling of a weight for rowstream_kernel. A tile holds the 128 row blocks of one
// (panel, unit) pair, split into up to four sections, each the same field of all 128 rows back to
// back: [panel][unit][section][row in panel][field bytes]. A section is described by where the
// field starts in the source, the distance between rows and between units there, and its length
// (e.g. Q6_K: ql, qh, scales, d out of one 210-byte block; an affine pack: codes, scales and
// biases out of three arrays). Rows past N are zero. Fields are 2-byte aligned at worst, so the
// copy moves 2 bytes at a time.
struct TileSrc {
  const uint8_t *base;   // field of row 0, unit 0
  long long row_bytes;   // source distance between rows
  int unit_stride;       // source distance between units of a row
  int field_bytes;       // bytes per row per unit
  int sec_off;           // section offset inside a tile
};

static __global__ void __launch_bounds__(256) prepare_tiles_kernel(TileSrc s0, TileSrc s1, TileSrc s2, TileSrc s3, int nsec,
                                                            long long N, int units, int tile_bytes,
                                                            uint8_t *__restrict__ dst) {
  const TileSrc src[4] = {s0, s1, s2, s3};
  const long long P = (N + kRowPanel - 1) / kRowPanel;
  const long long total = P * units * kRowPanel;  // (panel, unit, row) triples
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i % kRowPanel);
    const long long pu = i / kRowPanel;
    const int u = (int)(pu % units);
    const long long p = pu / units;
    const long long row = p * kRowPanel + r;
    uint8_t *tile = dst + pu * (long long)tile_bytes;
    for (int k = 0; k < nsec; ++k) {
      uint16_t *o = reinterpret_cast<uint16_t *>(tile + src[k].sec_off + (long long)r * src[k].field_bytes);
      const int n16 = src[k].field_bytes / 2;
      if (row < N) {
        const uint16_t *in = reinterpret_cast<const uint16_t *>(src[k].base + row * src[k].row_bytes +
                                                                (long long)u * src[k].unit_stride);
        for (int j = 0; j < n16; ++j) o[j] = in[j];
      } else {
        for (int j = 0; j < n16; ++j) o[j] = 0;
      }
    }
  }
}

}  // namespace ishi
