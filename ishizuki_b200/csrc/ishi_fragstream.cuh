// The warp-level verify-matmul kernel: y[m, n] = sum_k x[m, k] * w[n, k] for 1..8 activation rows
// on mma.sync (m16n8k16, weights on the M side, activation rows on the N side), with a CUDA-core
// variant for a single row.
//
// Why not tcgen05 here: eight activation rows fill an m16n8k16 fragment exactly, twenty-odd warps
// per SM decode in registers right beside the MMA, and on the same weights this kernel measures
// about twice as fast as the tcgen05 kernel (ishi_rowstream.cuh: 128 weight rows per instruction,
// four decode warps per CTA feeding tensor memory). That kernel stays for the formats that have
// no fragment decoder and for inputs too wide for this one's shared memory.
//
// Layout. The weight is re-tiled once, when the projection is created, into fragment order: a
// tile is 16 output rows x 256 k (one unit), stored as [16-byte piece][lane] so that every
// warp-wide 128-bit access is one contiguous 512-byte run, followed by a small per-row section
// (block scales). Lane (g = lane / 4, t = lane % 4) owns weight rows g and g + 8 of the tile and,
// in every k-step, the four k positions the format's decoder assigns to t. Same bytes as the raw
// weight, different order.
//
// Work. K is cut into S column ranges and the kernel is launched as thread-block clusters of S
// CTAs (S = 1: no cluster): CTA r of a cluster stages the activations of column range r into shared
// memory once, laid out as its format's decoder reads them, and all CTAs of a cluster walk the same
// run of 16-row panels, dealt to the clusters in equal contiguous runs. A CTA works on PP panels at a time ("panel lanes"), Wu warps
// per lane: warp (lane wp, position wu) takes panels wp, wp + PP, ... of the cluster's run and in
// each the units wu, wu + Wu, ... of the CTA's column range, streaming its tiles through a private
// ring in shared memory: one bulk async copy per tile (the copy engine, not the load/store unit,
// moves the bytes), completion counted on the ring slot's own mbarrier. No producer warp, no
// cross-warp wait on the data path.
//
// Reduction, without a CTA-wide barrier. With Wu = 1 a warp owns its panels whole and there is
// nothing to add up inside the CTA. Else a warp that has finished a panel parks its 16 x 8 partial
// tile in the lane's slot ring and bumps the slot's arrival counter; the warp that arrives last
// adds the lane's partials in warp order. With S > 1 it sends the CTA's partial panel into the
// shared memory of the panel's leader CTA (distributed shared memory, st.async counted on an
// mbarrier there); the leader's last-arriving warp waits for the S partials, adds them in rank
// order and writes y. Inbox slots are recycled two "generations" (G panels of a lane) later; a
// relaxed cluster barrier, arrived at the end of a generation and waited for one generation
// later, tells a sender that every leader is done with the slot it is about to overwrite. No
// global scratch, no atomics on values, every y element written once, the summation order fixed.
#pragma once
#include "ishi_stream.cuh"

namespace ishi {

constexpr int kFragRows = 16;
#ifndef ISHI_FRAG_MAX_WARPS
#define ISHI_FRAG_MAX_WARPS 24
#endif
// The kernel is compiled for two block sizes: up to kFragFewWarps warps with 96 registers per
// thread (the decoders' loads then run further ahead of their use), and up to kFragMaxWarps with 80.
// (A third one, 16 warps with 128 registers, measured no faster.)
constexpr int kFragMaxWarps = ISHI_FRAG_MAX_WARPS;
constexpr int kFragFewWarps = 20;
constexpr int kFragMaxRing = 4;   // most tiles per warp-private ring (FragArgs::ring of them are used:
                                  // one is decoded while the others are in flight)
constexpr int kFragMaxPanels = 24; // most panels a CTA works on in parallel (one warp each, then)
constexpr int kFragGroup = 4;     // most units per warp the planner considers
constexpr int kFragRed = 2;       // partial-tile slots per panel lane: a warp may run this many panels ahead of the slowest
constexpr int kFragMaxGen = 4;    // most panels of a lane per generation of inbox slots
constexpr int kFragMaxSplit = 8;  // portable cluster size
constexpr int kFragMaxPeers = 8;  // GPUs of one NVSwitch box

struct FragArgs {
  const uint8_t *tiles;  // [P][units][tile bytes]
  const __half *x;
  __half *y;
  long long ldy;
  int out_transposed;
  int M, N, K;
  int units, S, P, NC;  // NC clusters of S CTAs
  int Wu, PP, G;        // warps per panel, panels in parallel (Wu * PP warps per CTA), panels of a lane per inbox generation
  int ring;             // tiles per warp-private ring, 2 ... kFragMaxRing
  // ceil(2^32 / d) for d = S, NC, Wu, PP, or 0 for d = 1: see frag_div()
  unsigned inv_s, inv_nc, inv_wu, inv_pp;
  int umax;             // most units in a column range
  int group_size, scale_dtype;
  int *err;             // raised when a bounded wait gives up
  // Block Hadamard rotation of x while it is staged (0: none): xr = WHT_block(x * signs) / sqrt(block)
  int rot_block;           // a power of two, 8 ... 256
  const float *rot_signs;  // [K] or null
  // Gated pair (the weight was tiled with FragSrc::pair_rows): rows g and g + 8 of a panel are the
  // gate and the up row of output row 8 p + g, and the epilogue writes silu(gate) * up, N / 2 rows
  int swiglu;
  // Output exchange between the GPUs of an N-sharded projection (world = 0: none). Every rank holds
  // the whole output as [rows of all shards][8 or 16] fp16 at the same place of its exchange buffer; this
  // launch computes rows row_offset ... row_offset + N - 1 and stores them into every rank's copy
  // over NVLink. When all CTAs have stored, the rank writes seq into its arrival word on every rank.
  int world, rank;
  __half *peer_y[kFragMaxPeers];          // the output array in every rank's buffer ([rank]: the local one)
  int peer_ld;                            // fp16 values between its rows: 8, or 16 when the call has more than 8 rows
  unsigned *peer_flags[kFragMaxPeers];    // every rank's arrival words; this rank writes word [rank] of each
  unsigned *local_flags;                  // this rank's arrival words, one per rank
  unsigned *done;                         // CTAs of this launch that have stored their rows
  // The launches of an exchange are numbered on the device (so that a captured graph can be
  // replayed): *launch_no is the number of the last launch that completed on this rank; all ranks
  // issue the same sequence, so the numbers agree across ranks.
  unsigned *launch_no;
  int wait_previous;                      // first wait until every rank's previous launch has arrived here
  long long row_offset;
  unsigned long long *trace;              // diagnostic builds (-DISHI_TRACE): [CTA][warp][32] timestamps, else unused
};

// Diagnostic builds stamp the global nanosecond timer at the kernel's phase boundaries.
#ifdef ISHI_TRACE
#define ISHI_STAMP(slot)                                                                                   \
  do {                                                                                                     \
    if (a.trace && lane == 0) {                                                                            \
      unsigned long long t_;                                                                               \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)::"memory");                                    \
      a.trace[((size_t)blockIdx.x * kFragMaxWarps + warp) * 32 + (slot)] = t_;                             \
    }                                                                                                      \
  } while (0)
// ... and add up the clock cycles a warp spends in each part of its panel loop (slots 16 ... 23)
#define ISHI_CLOCK(var) const long long var = clock64()
#define ISHI_SPENT(slot, from, to)                                                                        \
  do {                                                                                                     \
    if (a.trace && lane == 0) a.trace[((size_t)blockIdx.x * kFragMaxWarps + warp) * 32 + (slot)] += (unsigned long long)((to) - (from)); \
  } while (0)
#else
#define ISHI_STAMP(slot) \
  do {                   \
  } while (0)
#define ISHI_CLOCK(var) \
  do {                  \
  } while (0)
#define ISHI_SPENT(slot, from, to) \
  do {                             \
  } while (0)
#endif

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
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t a) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(a) : "memory");
}
// (not volatile: callers tie the address to the barrier that publishes the data)
__device__ __forceinline__ float lds32f(uint32_t addr) {
  float v;
  asm("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
// the address of this CTA's shared-memory location addr in CTA rank of the cluster
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// 4 bytes into another CTA's shared memory; the bytes count as completed on that CTA's mbarrier
// when they have landed, so the reader needs no fence: it waits for the barrier's phase
__device__ __forceinline__ void st_async32(uint32_t addr, float v, uint32_t mbar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];" ::"r"(addr), "f"(v),
               "r"(mbar)
               : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// arrival without the release fence, which would wait for every copy and store in flight; the
// data that crosses CTAs here is published by mbarriers instead
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_relaxed() { asm volatile("barrier.cluster.wait.aligned;" ::: "memory"); }
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// n / d through inv = ceil(2^32 / d), exact for n * d < 2^32; inv = 0 stands for d = 1
__device__ __forceinline__ int frag_div(unsigned n, unsigned inv) { return inv ? (int)__umulhi(n, inv) : (int)n; }
__host__ inline unsigned frag_inverse(int d) { return d == 1 ? 0u : (unsigned)(((1ull << 32) + d - 1) / d); }

__host__ __device__ inline int frag_column_begin(int c, int units, int S) { return (c * units) / S; }
__host__ __device__ inline int frag_ring_stride(int tile_bytes) { return (tile_bytes + 127) & ~127; }

// shared memory of one CTA, in order: activations, the lanes' partial-tile slots, the inbox for the
// partial panels of the cluster's CTAs, a control block (inbox mbarriers, arrival counters,
// progress words, abort word), the warps' rings
// control block (PP <= 24, G <= 2): inbox mbarriers [PP][2G] @0, phases used of each [PP][2G] @768,
// arrival counters [PP][kFragRed] @1152, done [PP] @1344, abort @1440, ring mbarriers
// [warp][kFragMaxRing] @1472
constexpr uint32_t kFragCtrlBytes = 2304;
// xregion: the format's activation staging, umax * Fmt::kXBytes + Fmt::kExtraBytes
// (a panel lane of one warp parks nothing and has no slots)
__host__ __device__ inline size_t frag_smem_bytes(size_t xregion, int W, int PP, int G, int S, int tile_bytes, int ring) {
  return xregion + (W > PP ? (size_t)W * kFragRed * 512 : 0) + (S > 1 ? (size_t)PP * 2 * G * S * 512 : 0) + kFragCtrlBytes +
         (size_t)W * ring * frag_ring_stride(tile_bytes);
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(unsigned *p, unsigned v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// silu(gate) * up as the reference's MLP computes it on fp16 arrays (downProj(silu(gateProj(x)) *
// upProj(x)), Sources/IshizukiKit/Text/Attention.swift:251): the two products rounded to fp16,
// sigmoid, gate * sigmoid and the product with up each rounded to fp16 (one array per operation),
// the arithmetic itself in fp32. Returns the fp16 value as a float.
__device__ __forceinline__ float frag_swiglu(float gate, float up) {
  const float gf = __half2float(__float2half_rn(gate)), uf = __half2float(__float2half_rn(up));
  const float sig = __half2float(__float2half_rn(1.0f / (1.0f + expf(-gf))));
  const float act = __half2float(__float2half_rn(gf * sig));
  return __half2float(__float2half_rn(act * uf));
}

// One lane's part of panel p's finished 16 x 8 tile, in accumulator-fragment order: lane
// (g = lane / 4, t = lane % 4) holds v.x, v.y = weight row g, activation rows 2t, 2t + 1 and
// v.z, v.w = weight row g + 8, the same activation rows. Called by all 32 lanes of a warp.
// With an output exchange the four lanes of a weight row gather its eight values and one of them
// stores the 16 bytes into every rank's copy.
__device__ __forceinline__ void frag_write(const FragArgs &a, int p, int lane, float4 v) {
  const int g = lane >> 2, t = lane & 3;
  const long long n0 = (long long)p * kFragRows + g;
  if (a.swiglu) {
    // v.x, v.y: the gate row, v.z, v.w: the up row of output row 8 p + g
    v.x = frag_swiglu(v.x, v.z), v.y = frag_swiglu(v.y, v.w);
    const long long n = (long long)p * 8 + g;
    if (a.world > 0) {
      const __half2 h = __floats2half2_rn(v.x, v.y);
      const uint32_t ph = *reinterpret_cast<const uint32_t *>(&h);
      const int base = lane & ~3;
      uint4 row;
      row.x = __shfl_sync(0xffffffffu, ph, base), row.y = __shfl_sync(0xffffffffu, ph, base + 1);
      row.z = __shfl_sync(0xffffffffu, ph, base + 2), row.w = __shfl_sync(0xffffffffu, ph, base + 3);
      if (n < a.N / 2 && t < 2)  // lanes t = 0, 1 store to the even / odd ranks
        for (int q = t; q < a.world; q += 2) *reinterpret_cast<uint4 *>(a.peer_y[q] + (a.row_offset + n) * a.peer_ld) = row;
      return;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int m = 2 * t + i;
      if (n < a.N / 2 && m < a.M) {
        const __half h = __float2half_rn(i ? v.y : v.x);
        if (a.out_transposed) a.y[n * a.ldy + m] = h;
        else a.y[(long long)m * a.ldy + n] = h;
      }
    }
    return;
  }
  if (a.world > 0) {
    const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
    const uint32_t plo = *reinterpret_cast<const uint32_t *>(&lo), phi = *reinterpret_cast<const uint32_t *>(&hi);
    const int base = lane & ~3;
    uint4 rlo, rhi;
    rlo.x = __shfl_sync(0xffffffffu, plo, base), rlo.y = __shfl_sync(0xffffffffu, plo, base + 1);
    rlo.z = __shfl_sync(0xffffffffu, plo, base + 2), rlo.w = __shfl_sync(0xffffffffu, plo, base + 3);
    rhi.x = __shfl_sync(0xffffffffu, phi, base), rhi.y = __shfl_sync(0xffffffffu, phi, base + 1);
    rhi.z = __shfl_sync(0xffffffffu, phi, base + 2), rhi.w = __shfl_sync(0xffffffffu, phi, base + 3);
    // lanes t = 0, 1 store row g to the even / odd ranks, lanes t = 2, 3 row g + 8
    const long long n = n0 + ((t & 2) ? 8 : 0);
    if (n < a.N) {
      const uint4 row = (t & 2) ? rhi : rlo;
      for (int q = t & 1; q < a.world; q += 2) *reinterpret_cast<uint4 *>(a.peer_y[q] + (a.row_offset + n) * a.peer_ld) = row;
    }
    return;
  }
  const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long n = n0 + ((i & 2) ? 8 : 0);
    const int m = 2 * t + (i & 1);
    if (n < a.N && m < a.M) {
      const __half h = __float2half_rn(e[i]);
      if (a.out_transposed) a.y[n * a.ldy + m] = h;
      else a.y[(long long)m * a.ldy + n] = h;
    }
  }
}

// Eight consecutive activations of one row (this lane's k = 8 * lane ... 8 * lane + 7 of a
// 256-wide unit) through the block Hadamard rotation, all 32 lanes together. fp32 inside, radix-2
// stages h = 1, 2, 4 in the lane and h = 8 ... block / 2 across lanes, in that order and with the
// same roundings as hadamard_rotate_kernel, so the result is bit-identical to rotating first.
__device__ __forceinline__ uint4 frag_rotate8(uint4 v, int block, const float *signs, int lane) {
  float f[8];
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 p = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
    f[2 * i] = p.x;
    f[2 * i + 1] = p.y;
  }
  if (signs) {
    const float4 s0 = __ldg(reinterpret_cast<const float4 *>(signs)), s1 = __ldg(reinterpret_cast<const float4 *>(signs) + 1);
    const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __fmul_rn(f[i], s[i]);
  }
#pragma unroll
  for (int h = 1; h < 8; h <<= 1)
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (!(j & h)) {
        const float lo = f[j], hi = f[j + h];
        f[j] = __fadd_rn(lo, hi);
        f[j + h] = __fsub_rn(lo, hi);
      }
  for (int d = 1; d < block / 8; d <<= 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float o = __shfl_xor_sync(0xffffffffu, f[j], d);
      f[j] = (lane & d) ? __fsub_rn(o, f[j]) : __fadd_rn(f[j], o);
    }
  }
  const float scale = 1.0f / sqrtf((float)block);
  uint32_t r[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h2 = __halves2half2(__float2half_rn(__fmul_rn(f[2 * i], scale)), __float2half_rn(__fmul_rn(f[2 * i + 1], scale)));
    r[i] = *reinterpret_cast<const uint32_t *>(&h2);
  }
  return make_uint4(r[0], r[1], r[2], r[3]);
}

// 16 bytes into another CTA's shared memory; the bytes count as completed on that CTA's mbarrier
// when they have landed, so the reader needs no fence: it waits for the barrier's phase
__device__ __forceinline__ void st_async128(uint32_t addr, float4 v, uint32_t mbar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1,%2,%3,%4}, [%5];" ::"r"(addr),
               "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"(mbar)
               : "memory");
}

// MODE 0: tensor-core (rows 1..8); MODE 1: CUDA-core FMA for a single row. MAXW: most warps of a block.
template <class Fmt, int MODE, int MAXW>
__global__ void __launch_bounds__(MAXW * 32, 1) frag_kernel(const FragArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kTile = Fmt::kTileBytes;
  constexpr uint32_t kStride = (uint32_t)((kTile + 127) & ~127);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int S = a.S, Wu = a.Wu, PP = a.PP, G = a.G;
  const int W = Wu * PP;
  // This warp's position wu in its panel lane wp. The lanes are dealt round robin over the warps,
  // so that with 2 or 4 lanes all warps of an SM sub-partition (warp % 4) belong to one lane: the
  // scheduler's preference for its oldest warps then cannot starve a whole lane.
  const int wu = frag_div((unsigned)warp, a.inv_pp), wp = warp - wu * PP;

  const uint32_t xfrag = smem_u32(smem);                                   // [umax][Fmt::kXBytes], then Fmt::kExtraBytes
  const uint32_t red = xfrag + (uint32_t)a.umax * Fmt::kXBytes + Fmt::kExtraBytes;  // [PP][kFragRed][Wu][128 floats]
  const uint32_t inbox = red + (Wu > 1 ? (uint32_t)(W * kFragRed) * 512u : 0u);  // [PP][2G][S][128 floats]
  const uint32_t ctrl = inbox + (S > 1 ? (uint32_t)(PP * 2 * G * S) * 512u : 0u);
  const int R = a.ring;  // tiles in this warp's ring
  const uint32_t ring = ctrl + kFragCtrlBytes + (uint32_t)(warp * R) * kStride;
  uint8_t *ctrl_p = smem + (ctrl - xfrag);
  uint64_t *bars = reinterpret_cast<uint64_t *>(ctrl_p);                   // [PP][2G]
  int *cnt = reinterpret_cast<int *>(ctrl_p + 1152);                       // [PP][kFragRed] arrivals of the lane's warps
  volatile int *done = reinterpret_cast<volatile int *>(ctrl_p + 1344);    // [PP] panels of the lane whose partials were added
  volatile int *abort_word = reinterpret_cast<volatile int *>(ctrl_p + 1440);
  volatile int *uses = reinterpret_cast<volatile int *>(ctrl_p + 768);     // [PP][2G] completed phases of each inbox mbarrier

  // (divisions by multiplication: the host checks the ranges)
  const int cid = frag_div(blockIdx.x, a.inv_s);
  const int r = (int)blockIdx.x - cid * S;  // rank in the cluster = column range
  const int ub0 = frag_div((unsigned)(r * a.units), a.inv_s);  // = frag_column_begin(r, units, S)
  const int uc = frag_div((unsigned)((r + 1) * a.units), a.inv_s) - ub0;
  // the cluster's panels: pa .. pa + np - 1
  const int pa = frag_div((unsigned)cid * (unsigned)a.P, a.inv_nc);
  const int np = frag_div((unsigned)(cid + 1) * (unsigned)a.P, a.inv_nc) - pa;
  const int per = frag_div((unsigned)(uc - 1 - wu + Wu), a.inv_wu);  // units of a panel this warp owns: wu + i * Wu < uc
  const int contributors = min(Wu, uc);                              // warps of a lane that own a unit
  const int rounds = frag_div((unsigned)(np + PP - 1), a.inv_pp);    // panels of the fullest lane
  const int npw = np > wp ? frag_div((unsigned)(np - wp + PP - 1), a.inv_pp) : 0;  // panels this warp takes: wp, wp + PP, ...

  ISHI_STAMP(0);
  // Let the next kernel on the stream start its own prologue as SMs fall free.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (threadIdx.x < 32) {  // the control block, a word or a barrier per lane of warp 0
    for (int i = threadIdx.x; i < PP * 2 * G; i += 32) {
      mbar_init(bars + i, 1);
      uses[i] = 0;
    }
    for (int i = threadIdx.x; i < PP * kFragRed; i += 32) cnt[i] = 0;
    if ((int)threadIdx.x < PP) done[threadIdx.x] = 0;
    if (threadIdx.x == 0) *abort_word = 0;
    mbar_fence_init();
  }
  // Shared memory of another CTA may be written only once that CTA runs and has set up its
  // barriers: every CTA arrives here, and waits before its first panel.
  if (S > 1) cluster_arrive_relaxed();  // the init fence above is what the peers need; nothing else to publish yet

  // This warp's tile sequence: its panels in order, in each its units wu + qi * Wu. The fetch
  // cursor runs R - 1 tiles ahead of the compute cursor. Lane 0 issues the copies; every
  // lane keeps the cursor.
  const uint32_t wbar = ctrl + 1472u + (uint32_t)warp * kFragMaxRing * 8u;  // this warp's ring mbarriers
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < kFragMaxRing; ++i) mbar_init_u32(wbar + 8u * i, 1);
    mbar_fence_init();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the copy engine sees the barriers initialised
  }
  __syncwarp();
  int f_left = npw * per, f_qi = 0, f_idx = 0;
  uint32_t f_slot = ring;
  const uint8_t *f_src = a.tiles + ((long long)(pa + wp) * a.units + ub0 + wu) * (long long)kTile;
  const long long step_unit = (long long)Wu * kTile;
  const long long step_panel = ((long long)PP * a.units - (long long)per * Wu) * kTile;
  auto fetch = [&]() {
    bulk_g2s_if(f_left > 0 && lane == 0, f_slot, f_src, (uint32_t)kTile, wbar + 8u * f_idx);
    --f_left;
    f_src += step_unit;
    if (++f_qi == per) {
      f_qi = 0;
      f_src += step_panel;
    }
    f_slot += kStride;
    if (++f_idx == R) {
      f_idx = 0;
      f_slot = ring;
    }
  };
  // The weight tiles are written by no earlier kernel: their first copies go out at once.
  for (int i = 0; i < R - 1; ++i) fetch();

  Fmt::before_wait(a, xfrag);  // tables that do not depend on earlier launches

  // Warm L2 and the address translation with this CTA's slice of x. Only a hint: x may still be
  // written by the kernel before this one, its values are read after the wait below, through L2.
  for (int r = warp; r < a.M; r += (int)(blockDim.x >> 5)) {
    const char *row = reinterpret_cast<const char *>(a.x + (long long)r * a.K + (long long)ub0 * 256);
    for (int c = lane; c < uc * 4; c += 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(row + c * 128));
  }

  // x may be the output of the kernel before this one and y may still be read by it: wait for the
  // earlier kernels (returns at once unless this kernel was launched early).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  ISHI_STAMP(1);
  unsigned previous_launch = 0;
  if (a.world > 0) {
    previous_launch = *reinterpret_cast<volatile unsigned *>(a.launch_no);
    if (a.wait_previous && previous_launch != 0) {
      // ... and for the other GPUs: x may be rows they stored into this rank's exchange buffer
      if ((int)threadIdx.x < a.world) {
        bool ok = false;
        for (uint32_t i = 0; i < kWaitSpins && !ok; ++i) {
          ok = (int)(ld_acquire_sys(a.local_flags + threadIdx.x) - previous_launch) >= 0;
          if (!ok) __nanosleep(64);
        }
        if (!ok) *a.err = 2;  // give up: the result is wrong, the error word tells the host
      }
    }
  }
  __syncthreads();  // the control block is set up for every warp; the other GPUs' rows have arrived
  ISHI_STAMP(2);

  // activations of the column range into fragment order (all warps)
  Fmt::stage_x(a, xfrag, ub0, uc, [&]() { ISHI_STAMP(8); });
  ISHI_STAMP(3);
  __syncthreads();
  ISHI_STAMP(4);
  // shared-memory loads are plain asm the compiler may move; tie their addresses to the waits
  const uint32_t xf = stage_acquire(xfrag);

  if (S > 1) cluster_wait_relaxed();
  ISHI_STAMP(5);

  int arrived = 0, waited = 0;  // cluster barrier generations this thread has arrived at / waited for
  int gen = 0, gpos = 0;        // generation of inbox slots, position of the lane's panel in it
  uint32_t c_slot = ring, c_phase = 0;
  int c_idx = 0;
  for (int i = 0; i < rounds; ++i, ++gpos) {
    if (gpos == G) {
      gpos = 0;
      ++gen;
      if (S > 1) {
        // generation gen - 1 is finished here; generation gen reuses the inbox slots of gen - 2,
        // which every leader has read once all warps of the cluster have finished gen - 2
        if (arrived > waited) {
          cluster_wait_relaxed();
          ++waited;
        }
        cluster_arrive_relaxed();
        ++arrived;
      }
    }
    const int pi = wp + i * PP;  // the panel's index in the cluster's run
    if (pi >= np || per == 0) continue;

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    {
      int uq = wu;  // the unit's index in the column range
      for (int qi = 0; qi < per; ++qi) {
        ISHI_CLOCK(c0);
        if (!mbar_wait_u32(wbar + 8u * c_idx, c_phase, abort_word)) *a.err = 1;  // this slot has landed
        __syncwarp();  // every lane is done with the previous slot
        if (i == 0 && qi == 0) ISHI_STAMP(6);
        ISHI_CLOCK(c1);
        fetch();                         // refill the previous slot
        Fmt::template unit<MODE>(acc, a, stage_acquire(c_slot), xf, uq, g, t, lane);
        values_ready(acc[0], acc[1], acc[2], acc[3]);
        ISHI_CLOCK(c2);
        ISHI_SPENT(16, c0, c1);
        ISHI_SPENT(17, c1, c2);
        uq += Wu;
        c_slot += kStride;
        if (++c_idx == R) {
          c_idx = 0;
          c_slot = ring;
          c_phase ^= 1u;
        }
      }
      if (MODE == 1) {
        // single activation row: each lane holds partial dot products of rows g (acc[0]) and
        // g + 8 (acc[2]) over its own k positions; add across the four lanes of a row
        acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 1);
        acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 2);
        acc[2] += __shfl_xor_sync(0xffffffffu, acc[2], 1);
        acc[2] += __shfl_xor_sync(0xffffffffu, acc[2], 2);
        if (t != 0) acc[0] = acc[2] = 0.f;  // one copy per row enters the sums below (column m = 0)
        acc[1] = acc[3] = 0.f;
      }
    }
    if (i == 0) ISHI_STAMP(7);

    // park the partial tile; the warp of the lane that arrives last adds the lane's partials
    ISHI_CLOCK(c3);
    float4 sum = make_float4(acc[0], acc[1], acc[2], acc[3]);
    bool last = true;
    if (contributors > 1) {
      const int rs = i & (kFragRed - 1);
      const uint32_t slot = red + (uint32_t)((wp * kFragRed + rs) * Wu) * 512u;
      if (i >= kFragRed && done[wp] < i - kFragRed + 1) {
        // the slot still holds the partials of panel i - kFragRed of this lane
        bool ok = false;
        for (uint32_t spin = 0; spin < kWaitSpins && !ok; ++spin) {
          ok = done[wp] >= i - kFragRed + 1;
          if (!ok && *abort_word != 0) break;
        }
        if (!ok) {
          *abort_word = 1;
          *a.err = 1;
        }
      }
      sts128(stage_acquire(slot) + (uint32_t)(wu * 32 + lane) * 16u, sum);
      __syncwarp();
      int old = 0;
      if (lane == 0) {
        __threadfence_block();
        old = atomicAdd(cnt + wp * kFragRed + rs, 1);
      }
      old = __shfl_sync(0xffffffffu, old, 0);
      last = old == contributors - 1;
      if (last) {
        __threadfence_block();
        const uint32_t src = stage_acquire(slot) + (uint32_t)lane * 16u;
        sum = lds128f(src);
        for (int w = 1; w < contributors; ++w) {
          const float4 o = lds128f(src + (uint32_t)w * 512u);
          sum.x += o.x, sum.y += o.y, sum.z += o.z, sum.w += o.w;
        }
        values_ready(sum.x, sum.y, sum.z, sum.w);
        __syncwarp();
        if (lane == 0) {
          cnt[wp * kFragRed + rs] = 0;
          __threadfence_block();
          done[wp] = i + 1;
        }
      }
    }
    ISHI_CLOCK(c4);
    ISHI_SPENT(18, c3, c4);
    if (!last) continue;

    if (S == 1) {
      frag_write(a, pa + pi, lane, sum);
    } else {
      // the CTA's partial panel goes to the panel's leader, rank pi % S
      const int lead = pi - frag_div((unsigned)pi, a.inv_s) * S;
      const int is = wp * 2 * G + (gen & 1) * G + gpos;  // inbox slot
      const uint32_t bar = ctrl + (uint32_t)is * 8u;
      const uint32_t box = inbox + (uint32_t)(is * S) * 512u + (uint32_t)lane * 16u;
      if (lead == r) {
        if (lane == 0) mbar_arrive_expect_tx(bars + is, (uint32_t)S * 512u);
        __syncwarp();
      }
      st_async128(cluster_map(box + (uint32_t)r * 512u, (uint32_t)lead), sum, cluster_map(bar, (uint32_t)lead));
      ISHI_CLOCK(c5);
      ISHI_SPENT(19, c4, c5);
      if (lead == r) {
        // a CTA leads only some of the panels that map to this slot, so the barrier's phase is
        // counted here; the slot's next use is two generations away, behind a cluster barrier
        const uint32_t parity = (uint32_t)uses[is] & 1u;
        bool ok = mbar_try_wait_cluster(bar, parity);
        for (uint32_t spin = 0; spin < kWaitSpins && !ok; ++spin) {
          ok = mbar_try_wait_cluster(bar, parity);
          if (!ok && *abort_word != 0) break;
        }
        if (!ok) {  // give up: y of this panel stays wrong, the error word tells the host
          *abort_word = 1;
          *a.err = 1;
        } else {
          const uint32_t src = stage_acquire(box);
          float4 total = lds128f(src);
          for (int q = 1; q < S; ++q) {
            const float4 o = lds128f(src + (uint32_t)q * 512u);
            total.x += o.x, total.y += o.y, total.z += o.z, total.w += o.w;
          }
          frag_write(a, pa + pi, lane, total);
        }
        __syncwarp();
        if (lane == 0) uses[is] = (int)parity + 1;
        ISHI_CLOCK(c6);
        ISHI_SPENT(20, c5, c6);
      }
    }
  }
  ISHI_STAMP(24);
  if (S > 1) {
    // no CTA leaves while another may still send to it or read its barriers
    if (arrived > waited) cluster_wait_relaxed();
    cluster_arrive_relaxed();
    cluster_wait_relaxed();
  }
  ISHI_STAMP(27);
  if (a.world > 0) {
    // This CTA's rows are on their way to every rank; the last CTA of the launch announces them.
    // One thread fences for the CTA (the barrier orders the other threads' stores before it) at
    // device scope and counts the CTA done; the CTA that counts last has thereby synchronised
    // with every other CTA, so its one system-scope fence covers all their rows (fences are
    // cumulative) before it raises the arrival words. A system-scope fence in every CTA, with its
    // own stores still in flight, measured 1.6 us slower per launch.
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      const unsigned before = atomicAdd(a.done, 1u);
      if (before == gridDim.x - 1) {
        *reinterpret_cast<volatile unsigned *>(a.done) = 0u;  // for the next launch on this stream
        *reinterpret_cast<volatile unsigned *>(a.launch_no) = previous_launch + 1u;
        __threadfence_system();
        for (int q = 0; q < a.world; ++q) st_relaxed_sys(a.peer_flags[q] + a.rank, previous_launch + 1u);
      }
    }
  }
}

// waits (bounded) until every rank's arrival word has reached this rank's latest launch
static __global__ void peer_wait_kernel(const unsigned *local_flags, int world, const unsigned *launch_no, int *err) {
  if ((int)threadIdx.x < world) {
    const unsigned seq = *reinterpret_cast<const volatile unsigned *>(launch_no);
    bool ok = false;
    for (uint32_t i = 0; i < kWaitSpins && !ok; ++i) {
      ok = (int)(ld_acquire_sys(local_flags + threadIdx.x) - seq) >= 0;
      if (!ok) __nanosleep(64);
    }
    if (!ok) *err = 2;
  }
}

// The exchange for products of the other kernels: rows [first, first + n) of this rank's own
// [.][8] array (just written by the product) go to every other rank's copy, columns past M
// cleared; then the same publication as in frag_kernel (last CTA: one system-scope fence, the
// launch number into this rank's arrival word on every rank).
struct PublishArgs {
  __half *peer_y[kFragMaxPeers];
  unsigned *peer_flags[kFragMaxPeers];
  unsigned *done, *launch_no;
  long long first, n;
  int world, rank, M;
};
static __global__ void __launch_bounds__(256) publish_rows_kernel(const PublishArgs a) {
  const unsigned previous_launch = *reinterpret_cast<volatile unsigned *>(a.launch_no);
  uint4 *mine = reinterpret_cast<uint4 *>(a.peer_y[a.rank]) + a.first;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += (long long)gridDim.x * blockDim.x) {
    uint4 v = mine[i];
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (2 * j >= a.M) w[j] = 0u;
      else if (2 * j + 1 >= a.M) w[j] &= 0xffffu;
    }
    v = make_uint4(w[0], w[1], w[2], w[3]);
    for (int q = 0; q < a.world; ++q) (reinterpret_cast<uint4 *>(a.peer_y[q]) + a.first)[i] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned before = atomicAdd(a.done, 1u);
    if (before == gridDim.x - 1) {
      *reinterpret_cast<volatile unsigned *>(a.done) = 0u;
      *reinterpret_cast<volatile unsigned *>(a.launch_no) = previous_launch + 1u;
      __threadfence_system();
      for (int q = 0; q < a.world; ++q) st_relaxed_sys(a.peer_flags[q] + a.rank, previous_launch + 1u);
    }
  }
}

// One-time re-tiling into fragment order: Fmt::tile_halfword says which 2 bytes of the source
// land at halfword hw of tile (p, u). Rows past N read as zero. The source may be several weights
// of the same format and input width stacked along the output rows (projections that share their
// input, fused into one launch): segment i holds rows first_row[i] ... first_row[i + 1] - 1.
constexpr int kFragMaxSegments = 4;
struct FragSrc {
  const uint8_t *w[kFragMaxSegments], *scales[kFragMaxSegments], *biases[kFragMaxSegments];
  long long first_row[kFragMaxSegments + 1];
  int segments;
  long long w_row_bytes, s_row_bytes;  // distance between rows
  long long N;
  int group_size, scale_bytes;
  // Two segments of equal height interleaved by eights instead of stacked: rows 0-7 of panel p are
  // rows 8 p ... 8 p + 7 of segment 0, rows 8-15 the same rows of segment 1, so that one
  // accumulator fragment holds a row of each (see FragArgs::swiglu).
  int pair_rows;
};

// which segment holds output row `row` (< N), and the row's index inside it
__device__ __forceinline__ int frag_segment(const FragSrc &s, long long row, long long *local) {
  if (s.pair_rows) {
    *local = (row >> 4) * 8 + (row & 7);
    return (int)(row >> 3) & 1;
  }
  int i = 0;
  while (i + 1 < s.segments && row >= s.first_row[i + 1]) ++i;
  *local = row - s.first_row[i];
  return i;
}

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
