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
// Work. K is cut into S column ranges and the kernel is launched as thread-block clusters of S
// CTAs: CTA r of a cluster stages the activations of column range r into shared memory once, in
// fragment order, and all CTAs of a cluster walk the same run of 16-row panels, dealt to the
// clusters in equal contiguous runs. Inside a CTA warp w takes the units u = w, w + W, ... of every
// panel and streams its tiles through a private ring in shared memory with cp.async (16 bytes per
// lane): no producer warp, no cross-warp wait on the data path. The warps meet once per group of
// panels (a CTA barrier) to add their partial tiles; the CTA's partial panel then goes into the
// shared memory of the panel's leader CTA (distributed shared memory), and after a cluster
// barrier, whose wait is deferred by one group so that it overlaps the next group's tiles, the
// leader adds the S partials in rank order and writes y. No global scratch, no atomics, every y
// element written once, the summation order fixed.
#pragma once
#include "ishi_stream.cuh"

namespace ishi {

constexpr int kFragRows = 16;
constexpr int kFragMaxWarps = 20;
constexpr int kFragRing = 3;      // tiles per warp-private ring: two in flight while one is decoded
constexpr int kFragGroup = 4;     // most panels of one warp between two CTA barriers
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
  int Wu, PP, SPW;      // warps per panel, panels in parallel (1, 2 or 4; Wu * PP warps per CTA), panels per warp and group
  int pp_shift;         // log2(PP)
  // ceil(2^32 / d) for d = S, NC, Wu, or 0 for d = 1: see frag_div()
  unsigned inv_s, inv_nc, inv_wu;
  int umax;             // most units in a column range
  int group_size, scale_dtype;
  int *err;             // raised when a bounded wait gives up
  // Block Hadamard rotation of x while it is staged (0: none): xr = WHT_block(x * signs) / sqrt(block)
  int rot_block;           // a power of two, 8 ... 256
  const float *rot_signs;  // [K] or null
  // Output exchange between the GPUs of an N-sharded projection (world = 0: none). Every rank holds
  // the whole output as [rows of all shards][8] fp16 at the same place of its exchange buffer; this
  // launch computes rows row_offset ... row_offset + N - 1 and stores them into every rank's copy
  // over NVLink. When all CTAs have stored, the rank writes seq into its arrival word on every rank.
  int world, rank;
  __half *peer_y[kFragMaxPeers];          // the output array in every rank's buffer ([rank]: the local one)
  unsigned *peer_flags[kFragMaxPeers];    // every rank's arrival words; this rank writes word [rank] of each
  unsigned *local_flags;                  // this rank's arrival words, one per rank
  unsigned *done;                         // CTAs of this launch that have stored their rows
  // The launches of an exchange are numbered on the device (so that a captured graph can be
  // replayed): *launch_no is the number of the last launch that completed on this rank; all ranks
  // issue the same sequence, so the numbers agree across ranks.
  unsigned *launch_no;
  int wait_previous;                      // first wait until every rank's previous launch has arrived here
  long long row_offset;
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

// shared memory of one CTA, in order: activations, partial tiles of the warps, partial panels of
// the cluster's CTAs, two mbarriers and an abort word, the warps' rings
__host__ __device__ inline size_t frag_smem_bytes(int umax, int xbytes, int W, int PP, int SPW, int S, int tile_bytes) {
  return (size_t)umax * xbytes + (size_t)W * SPW * 512 + 2 * (size_t)SPW * PP * S * 512 + 128 +
         (size_t)W * kFragRing * frag_ring_stride(tile_bytes);
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(unsigned *p, unsigned v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// element idx of panel p in accumulator-fragment order: lane idx / 4 (g = lane / 4, t = lane % 4),
// register e = idx % 4 -> weight row g + 8 * (e / 2), activation row 2t + e % 2.
// With an output exchange the 32 lanes of a warp hold 32 consecutive elements (two weight rows
// g, two rows g + 8, eight activation rows each): they gather each row's eight values in one lane,
// which stores the 16 bytes into every rank's copy.
__device__ __forceinline__ void frag_write(const FragArgs &a, int p, int idx, float v) {
  if (a.world > 0) {
    const uint32_t mine = __half_as_ushort(__float2half_rn(v));
    const uint32_t pair = mine | (__shfl_down_sync(0xffffffffu, mine, 1) << 16);  // activation rows 2t, 2t + 1 (even idx)
    const uint32_t w1 = __shfl_down_sync(0xffffffffu, pair, 4), w2 = __shfl_down_sync(0xffffffffu, pair, 8);
    const uint32_t w3 = __shfl_down_sync(0xffffffffu, pair, 12);
    if ((idx & 13) == 0) {  // t = 0 and an even register: weight row g + 8 * ((idx >> 1) & 1)
      const long long n = (long long)p * kFragRows + (idx >> 4) + ((idx & 2) ? 8 : 0);
      if (n < a.N) {
        const uint4 row = make_uint4(pair, w1, w2, w3);
        for (int q = 0; q < a.world; ++q) *reinterpret_cast<uint4 *>(a.peer_y[q] + (a.row_offset + n) * 8) = row;
      }
    }
    return;
  }
  const int ln = idx >> 2, e = idx & 3;
  const long long n = (long long)p * kFragRows + (ln >> 2) + ((e & 2) ? 8 : 0);
  const int m = 2 * (ln & 3) + (e & 1);
  if (n < a.N && m < a.M) {
    const __half h = __float2half_rn(v);
    if (a.out_transposed) a.y[n * a.ldy + m] = h;
    else a.y[(long long)m * a.ldy + n] = h;
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

// sum of n <= MAX floats at addr, addr + stride, ...: all loads are issued before the first add, so
// the latency of shared memory is paid once
template <int MAX>
__device__ __forceinline__ float lds_sum_upto(uint32_t addr, uint32_t stride, int n) {
  float v[MAX];
#pragma unroll
  for (int i = 0; i < MAX; ++i) v[i] = i < n ? lds32f(addr + (uint32_t)i * stride) : 0.f;
#pragma unroll
  for (int w = 1; w < MAX; w *= 2)
#pragma unroll
    for (int i = 0; i + w < MAX; i += 2 * w) v[i] += v[i + w];
  return v[0];
}
__device__ __forceinline__ float lds_sum(uint32_t addr, uint32_t stride, int n) {
  if (n <= 4) return lds_sum_upto<4>(addr, stride, n);
  if (n <= 8) return lds_sum_upto<8>(addr, stride, n);
  return lds_sum_upto<kFragMaxWarps>(addr, stride, n);
}

// MODE 0: tensor-core (rows 1..8); MODE 1: CUDA-core FMA for a single row.
template <class Fmt, int MODE>
__global__ void __launch_bounds__(kFragMaxWarps * 32, 1) frag_kernel(const FragArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kTile = Fmt::kTileBytes;
  constexpr uint32_t kStride = (uint32_t)((kTile + 127) & ~127);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int S = a.S, Wu = a.Wu, PP = a.PP, SPW = a.SPW, pp_shift = a.pp_shift;
  const int W = Wu * PP, SP = SPW * PP;
  const int wp = frag_div((unsigned)warp, a.inv_wu), wu = warp - wp * Wu;  // this warp's panel lane and unit lane

  const uint32_t xfrag = smem_u32(smem);                          // [umax][Fmt::kXBytes]
  const uint32_t red = xfrag + (uint32_t)a.umax * Fmt::kXBytes;   // [W][SPW][128 floats]
  const uint32_t inbox = red + (uint32_t)(W * SPW) * 512u;        // [2][SP][S][128 floats]
  const uint32_t full = inbox + 2u * (uint32_t)(SP * S) * 512u;   // two mbarriers (one per inbox half), the abort word
  const uint32_t ring = full + 128u + (uint32_t)warp * kFragRing * kStride;
  uint64_t *full_p = reinterpret_cast<uint64_t *>(smem + (full - xfrag));
  volatile int *abort_word = reinterpret_cast<volatile int *>(full_p + 2);
  const uint32_t ring_end = ring + kFragRing * kStride;

  // (divisions by multiplication: the host checks the ranges)
  const int cid = frag_div(blockIdx.x, a.inv_s);
  const int r = (int)blockIdx.x - cid * S;  // rank in the cluster = column range
  const int ub0 = frag_div((unsigned)(r * a.units), a.inv_s);  // = frag_column_begin(r, units, S)
  const int uc = frag_div((unsigned)((r + 1) * a.units), a.inv_s) - ub0;
  // the cluster's panels: pa .. pa + np - 1
  const int pa = frag_div((unsigned)cid * (unsigned)a.P, a.inv_nc);
  const int np = frag_div((unsigned)(cid + 1) * (unsigned)a.P, a.inv_nc) - pa;
  const int per = frag_div((unsigned)(uc - 1 - wu + Wu), a.inv_wu);  // units of a panel this warp owns: wu + i * Wu < uc
  const int npw = np > wp ? (np - wp + PP - 1) >> pp_shift : 0;           // panels this warp takes: wp, wp + PP, ...

  // Let the next kernel on the stream start its own prologue as SMs fall free.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // Shared memory of another CTA may be written only once that CTA runs and has set up its
  // barriers: every CTA arrives here, and waits before the first group.
  if (S > 1) {
    if (threadIdx.x == 0) {
      mbar_init(full_p, 1);
      mbar_init(full_p + 1, 1);
      *abort_word = 0;
      mbar_fence_init();
    }
    cluster_arrive_relaxed();  // the init fence above is what the peers need; nothing else to publish yet
  }

  // This warp's tile sequence: its panels in order, in each its units wu + qi * Wu. The fetch
  // cursor runs kFragRing - 1 tiles ahead of the compute cursor.
  int f_left = npw * per, f_qi = 0;
  uint32_t f_slot = ring + (uint32_t)lane * 16u;  // this lane's 16 bytes of every 512
  const uint32_t f_end = ring_end + (uint32_t)lane * 16u;
  const uint8_t *f_src = a.tiles + ((long long)(pa + wp) * a.units + ub0 + wu) * (long long)kTile + lane * 16;
  const long long step_unit = (long long)Wu * kTile;
  const long long step_panel = ((long long)PP * a.units - (long long)per * Wu) * kTile;
  auto fetch = [&]() {
    if (f_left > 0) {
#pragma unroll
      for (int o = 0; o + 512 <= kTile; o += 512) cp_async16(f_slot + o, f_src + o);
      if ((kTile & 511) != 0 && lane * 16 < (kTile & 511)) cp_async16(f_slot + (kTile & ~511), f_src + (kTile & ~511));
    }
    cp_async_commit();  // one group per slot, present or not, so the wait below counts slots
    --f_left;
    f_src += step_unit;
    if (++f_qi == per) {
      f_qi = 0;
      f_src += step_panel;
    }
    f_slot += kStride;
    if (f_slot == f_end) f_slot -= kFragRing * kStride;
  };
#pragma unroll
  for (int i = 0; i < kFragRing - 1; ++i) fetch();

  // Everything above reads only the weight tiles. x may be the output of the kernel before this
  // one and y may still be read by it: wait for the earlier kernels (returns at once unless this
  // kernel was launched early).
  asm volatile("griddepcontrol.wait;" ::: "memory");
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
      __syncthreads();
    }
  }

  // activations of the column range into fragment order (all warps), while the first tiles fly
  Fmt::stage_x(a, xfrag, ub0, uc);
  __syncthreads();
  // shared-memory loads are plain asm the compiler may move; tie their addresses to the waits
  const uint32_t xf = stage_acquire(xfrag) + (uint32_t)wu * Fmt::kXBytes;

  if (S > 1) cluster_wait_relaxed();

  // the leader of a group's panel pn: rank pn % S
  auto leader_of = [&](int pn) -> int { return pn - frag_div((unsigned)pn, a.inv_s) * S; };
  // the leaders' part of group gi: wait for the S partial panels, add them in rank order, write y
  auto finish_group = [&](int gi) {
    const uint32_t bar = full + (uint32_t)(gi & 1) * 8u, parity = (uint32_t)(gi >> 1) & 1u;
    if (!mbar_try_wait_cluster(bar, parity)) {
      bool ok = false;
      for (uint32_t i = 0; i < kWaitSpins && !ok; ++i) {
        ok = mbar_try_wait_cluster(bar, parity);
        if (!ok && *abort_word != 0) break;
      }
      if (!ok) {  // give up: y of this group stays wrong, the error word tells the host
        *abort_word = 1;
        *a.err = 1;
        return;
      }
    }
    const uint32_t ib = stage_acquire(inbox) + (uint32_t)((gi & 1) * SP * S) * 512u;
    for (int f = threadIdx.x; f < SP * 128; f += blockDim.x) {
      const int pn = f >> 7, idx = f & 127, pi = gi * SP + pn;
      if (pi >= np || leader_of(pn) != r) continue;
      frag_write(a, pa + pi, idx, lds_sum(ib + (uint32_t)(pn * S * 128 + idx) * 4u, 512u, S));
    }
  };

  const int ngroups = (np + SP - 1) / SP;
  uint32_t c_slot = ring;
  for (int gi = 0; gi < ngroups; ++gi) {
    // this warp's panels of the group, one after the other; each partial tile goes straight to the
    // reduction buffer (the barrier at the end of the previous group freed it)
    for (int k = 0; k < SPW; ++k) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      if (gi * SP + k * PP + wp < np) {
        uint32_t xq = xf;
        for (int qi = 0; qi < per; ++qi) {
          cp_async_wait<kFragRing - 2>();  // this slot has landed (the younger ones may still be in flight)
          __syncwarp();                    // ... for every lane, and every lane is done with the previous slot
          fetch();                         // refill the previous slot
          Fmt::template unit<MODE>(acc, a, stage_acquire(c_slot), xq, g, t, lane);
          values_ready(acc[0], acc[1], acc[2], acc[3]);
          xq += (uint32_t)Wu * Fmt::kXBytes;
          c_slot += kStride;
          if (c_slot == ring_end) c_slot = ring;
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
      sts128(red + ((uint32_t)(warp * SPW + k) * 32u + lane) * 16u, make_float4(acc[0], acc[1], acc[2], acc[3]));
    }

    // add the warps' partial tiles (all threads, one output element each)
    __syncthreads();
    if (S > 1 && gi > 0) {
      cluster_wait_relaxed();  // every CTA has read what it led of group gi - 2: that inbox half is free
      finish_group(gi - 1);
    }
    if (S > 1 && threadIdx.x == 0) {
      // what this CTA will receive for group gi: S partial panels for every panel it leads
      // (panels r, r + S, ... of the group, as far as the group goes)
      const int left = min(SP, np - gi * SP);
      const int led = left > r ? (left - r + S - 1) / S : 0;
      mbar_arrive_expect_tx(full_p + (gi & 1), (uint32_t)(led * S) * 512u);
    }
    {
      const uint32_t rbs = stage_acquire(red);
      for (int f = threadIdx.x; f < SP * 128; f += blockDim.x) {
        const int pn = f >> 7, idx = f & 127, pi = gi * SP + pn;
        if (pi >= np) continue;
        const uint32_t src = rbs + (uint32_t)(((pn & (PP - 1)) * Wu * SPW + (pn >> pp_shift)) * 128 + idx) * 4u;
        const float sum = lds_sum(src, (uint32_t)SPW * 512u, Wu);
        if (S == 1) {
          frag_write(a, pa + pi, idx, sum);
        } else {
          const uint32_t lead = (uint32_t)leader_of(pn);
          const uint32_t mine = inbox + (uint32_t)((((gi & 1) * SP + pn) * S + r) * 128 + idx) * 4u;
          st_async32(cluster_map(mine, lead), sum, cluster_map(full + (uint32_t)(gi & 1) * 8u, lead));
        }
      }
    }
    if (S > 1) cluster_arrive_relaxed();
    __syncthreads();  // every thread has read the reduction buffer: the next group may write it
  }
  if (S > 1) {
    if (ngroups > 0) {
      cluster_wait_relaxed();
      finish_group(ngroups - 1);
    }
    // no CTA leaves while another may still send to it or read its barriers
    cluster_arrive_relaxed();
    cluster_wait_relaxed();
  }
  cp_async_wait<0>();
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
__global__ void peer_wait_kernel(const unsigned *local_flags, int world, const unsigned *launch_no, int *err) {
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
