// C ABI of the verify-matmul library: argument validation, per-shape launch plans, the one-time
// re-tiling of weights and the kernel launches. No torch, no NCCL, no CPU fallback: a shape
// without a kernel is an error status.
#include <cuda_runtime.h>

#include <algorithm>
#include <array>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include <new>
#include <vector>

#include "../../include/ishizuki_cuda.h"
#include "dequant.cuh"
#include "ishi_kernels.h"

using namespace ishi;

namespace ishi {
// the per-format kernel tables (frag_*.cu, row_*.cu)
const FragOps *frag_ops_q4k();
const FragOps *frag_ops_q6k();
const FragOps *frag_ops_iq2xs();
const FragOps *frag_ops_iq4xs();
const FragOps *frag_ops_iq2xxs();
const FragOps *frag_ops_iq2s();
const FragOps *frag_ops_iq3xxs();
const FragOps *frag_ops_iq3s();
const FragOps *frag_ops_q2k();
const FragOps *frag_ops_iq1s();
const FragOps *frag_ops_iq1m();
const FragOps *frag_ops_ggml_a(int type);
const FragOps *frag_ops_ggml_b(int type);
const FragOps *frag_ops_affine4(int group_size, bool bf16);
const FragOps *frag_ops_affine2(int group_size, bool bf16);
const RowOps *row_ops_ggml(int type);
const RowOps *row_ops_affine(int bits);
}  // namespace ishi

namespace {

constexpr int kSmemPerSm = 227 * 1024;

struct Workspace {
  float *scratch = nullptr;
  unsigned int *counters = nullptr;
  uint8_t *tiles = nullptr;  // kernel-level calls re-tile the weight here on every call
  size_t scratch_floats = 0, n_counters = 0, tiles_bytes = 0;
  mutable unsigned epoch = 0;  // the context's time-out count when the counters were last known to be zero
};

// Internal format id: the GGML type number, or 100 + bits for an affine pack.
int format_of(const ishi_weight_desc &d) { return d.kind == ISHI_KIND_GGML ? d.ggml_type : 100 + d.bits; }

struct RowPlan {
  bool ok = false;
  int units = 0, P = 0, SL = 2, kc = 2, nstages = 2, x_off = 0, bmin_off = 0, xs_off = 0, stage_bytes = 0;
  int grid = 0, nsec = 0, table_bytes = 0;
  int tile_bytes = 0, sec_off[4] = {0, 0, 0, 0}, sec_bytes[4] = {0, 0, 0, 0};
  TileSrc src[4];
  size_t smem = 0, scratch_floats = 0, counters = 0, tiles_bytes = 0;
};

// Launch plan of the warp-level kernel (fragment-order tiles, 16-row panels, clusters of S CTAs).
struct FragPlan {
  bool ok = false;
  const FragOps *ops = nullptr;  // the format's kernels
  int units = 0, S = 1, P = 0, NC = 1, Wu = 1, PP = 1, G = 1, ring = 3, umax = 0, tile_bytes = 0;
  size_t smem = 0, tiles_bytes = 0;
  double cost = 0;
};

}  // namespace

struct ishi_ctx {
  int device = 0;
  int sm_count = 0;
  int smem_optin = 0;
  int route = ISHI_ROUTE_AUTO;
  int crossover_rows = 0;
  int *err_host = nullptr;  // mapped pinned word the kernels raise on a timed-out wait
  unsigned timeout_epoch = 0;  // time-outs seen by ishi_ctx_poll: arrival counters from before may be stale
  int *err_dev = nullptr;
  Workspace ws;                             // for the kernel-level entry points
  void *pin_x = nullptr, *pin_y = nullptr;  // pinned staging for apply_host
  void *dev_x = nullptr, *dev_y = nullptr;
  size_t pin_x_bytes = 0, pin_y_bytes = 0;
  __half *exl3_x = nullptr;  // ishi_exl3_apply: rotated activations [16][k] and fp32 products [16][n]
  float *exl3_y = nullptr;
  size_t exl3_x_cap = 0, exl3_y_cap = 0;
  // apply_host_batch: its two copy streams and the events that order them against the caller's stream
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  std::vector<cudaEvent_t> ev_in, ev_done;
  cudaEvent_t ev_begin = nullptr, ev_end = nullptr;
  std::mutex lock;
  // launch plans already measured on this device, by (format's kernels, output rows, input width):
  // {K split, warps per panel, panels in parallel, ring}
  std::map<std::tuple<const void *, long long, long long>, std::array<int, 4>> tuned;
  char last_error[256] = {0};
};

struct ishi_projection {
  ishi_ctx *ctx = nullptr;
  ishi_weight_desc d;
  int fmt = 0;
  RowPlan plan;          // tcgen05 kernel (formats without a fragment decoder)
  FragPlan frag;         // warp-level kernel
  bool generic = false;  // neither: the one-warp-per-row kernel reads a plain copy of the blocks (ws.tiles)
  bool gated = false;    // gate and up interleaved by eights, the kernel's epilogue writes silu(gate) * up: d.n / 2 output rows
  __half *logits = nullptr;  // [16][n] of apply_argmax, allocated by its first call
  Workspace ws;          // this projection's own scratch and tiled weight: apply never allocates
  __half *xr = nullptr;  // rotated activations [16][k] when the pack is rotated
  __half *host_x = nullptr, *host_y = nullptr;  // device staging of apply_host_async: [16][k], [16][n]
  int64_t weight_bytes = 0;
};

namespace {

// output rows the caller sees
int64_t out_rows(const ishi_projection *p) { return p->gated ? p->d.n / 2 : p->d.n; }

ishi_status fail(ishi_ctx *ctx, ishi_status s, const char *fmt, ...) {
  if (ctx) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(ctx->last_error, sizeof(ctx->last_error), fmt, ap);
    va_end(ap);
  }
  return s;
}

#define ISHI_CUDA(ctx, call)                                                                       \
  do {                                                                                             \
    cudaError_t e_ = (call);                                                                       \
    if (e_ != cudaSuccess) return fail(ctx, ISHI_E_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
  } while (0)

int type_size(int t) { return ggml_type_size(t); }

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// The reference's shape guards plus this library's own (Sources/IshizukiKit/Core/VerifyMatmul.swift
// :78-87, Sources/IshizukiKit/Core/GGMLKernels.swift:181-189,223-230). Fills weight_bytes.
ishi_status check_desc(ishi_ctx *ctx, const ishi_weight_desc &d, int64_t *weight_bytes) {
  if (!d.weight_dev || (reinterpret_cast<uintptr_t>(d.weight_dev) & 3u))
    return fail(ctx, ISHI_E_INVALID, "weight pointer null or not 4-byte aligned");
  if (d.n <= 0 || d.k <= 0) return fail(ctx, ISHI_E_SHAPE, "n and k must be positive");
  if (d.n > (1ll << 31) - 256 || d.k > (1ll << 30)) return fail(ctx, ISHI_E_SHAPE, "shape too large");
  if (d.k % 256 != 0) return fail(ctx, ISHI_E_SHAPE, "k %lld is not a whole number of 256-wide blocks", (long long)d.k);
  if (d.hadamard_block != 0) {
    const int b = d.hadamard_block;
    if (b < 0 || (b & (b - 1)) != 0 || b > 8192 || d.k % b != 0)
      return fail(ctx, ISHI_E_SHAPE, "Hadamard block %d does not divide input width %lld", b, (long long)d.k);
  }
  // the product kernel reads the rotation signs four at a time
  if (d.hadamard_block != 0 && d.signs_dev && !aligned16(d.signs_dev))
    return fail(ctx, ISHI_E_INVALID, "rotation signs must be 16-byte aligned");
  int64_t bytes = 0, total = 0;
  if (d.kind == ISHI_KIND_GGML) {
    const int ts = type_size(d.ggml_type);
    if (ts == 0) return fail(ctx, ISHI_E_UNSUPPORTED, "GGML type %d has no decoder here", d.ggml_type);
    bytes = total = d.n * (d.k / 256) * ts;
  } else if (d.kind == ISHI_KIND_AFFINE) {
    if (d.bits < 2 || d.bits > 8) return fail(ctx, ISHI_E_SHAPE, "affine width %d outside 2...8", d.bits);
    if (d.bits != 2 && d.bits != 4 && d.bits != 8)
      return fail(ctx, ISHI_E_UNSUPPORTED, "affine width %d has no kernel here", d.bits);
    if (d.group_size != 32 && d.group_size != 64 && d.group_size != 128)
      return fail(ctx, ISHI_E_SHAPE, "group size %d outside {32, 64, 128}", d.group_size);
    if (d.scale_dtype < ISHI_DT_F16 || d.scale_dtype > ISHI_DT_F32) return fail(ctx, ISHI_E_INVALID, "bad scale dtype");
    if (!d.scales_dev || !d.biases_dev || (reinterpret_cast<uintptr_t>(d.scales_dev) & 3u) ||
        (reinterpret_cast<uintptr_t>(d.biases_dev) & 3u))
      return fail(ctx, ISHI_E_INVALID, "scales/biases null or misaligned");
    const int sb = d.scale_dtype == ISHI_DT_F32 ? 4 : 2;
    bytes = d.n * d.k * d.bits / 8;
    total = bytes + 2 * d.n * (d.k / d.group_size) * sb;
  } else {
    return fail(ctx, ISHI_E_INVALID, "bad weight kind %d", d.kind);
  }
  if (d.weight_bytes < bytes)
    return fail(ctx, ISHI_E_SHAPE, "weight buffer holds %lld bytes, shape needs %lld", (long long)d.weight_bytes,
                (long long)bytes);
  *weight_bytes = total;
  return ISHI_OK;
}

const RowOps *row_ops(int fmt) { return fmt >= 100 ? row_ops_affine(fmt - 100) : row_ops_ggml(fmt); }

// Sections of a tile for each format: which field of the source goes where.
void describe_sections(const ishi_weight_desc &d, RowPlan *pl) {
  const uint8_t *w = static_cast<const uint8_t *>(d.weight_dev);
  const long long units = d.k / 256;
  auto sec = [&](int i, const uint8_t *base, long long row_bytes, int unit_stride, int field) {
    pl->src[i].base = base;
    pl->src[i].row_bytes = row_bytes;
    pl->src[i].unit_stride = unit_stride;
    pl->src[i].field_bytes = field;
  };
  memset(pl->src, 0, sizeof(pl->src));
  if (d.kind == ISHI_KIND_GGML) {
    const int ts = type_size(d.ggml_type);
    const long long rb = units * ts;
    switch (d.ggml_type) {
      case ISHI_GGML_Q4_K:
        pl->nsec = 1;
        sec(0, w, rb, ts, 144);
        break;
      case ISHI_GGML_Q6_K:
        pl->nsec = 4;
        sec(0, w, rb, ts, 128);       // ql
        sec(1, w + 128, rb, ts, 64);  // qh
        sec(2, w + 192, rb, ts, 16);  // scales
        sec(3, w + 208, rb, ts, 2);   // d
        break;
      default:  // IQ2_XS
        pl->nsec = 3;
        sec(0, w + 2, rb, ts, 64);  // index words
        sec(1, w + 66, rb, ts, 8);  // scale bytes
        sec(2, w, rb, ts, 2);       // d
        break;
    }
  } else {
    const int sb = d.scale_dtype == ISHI_DT_F32 ? 4 : 2;
    const int per_unit = 256 / d.group_size;
    pl->nsec = 3;
    sec(0, w, d.k * d.bits / 8, 32 * d.bits, 32 * d.bits);
    sec(1, static_cast<const uint8_t *>(d.scales_dev), (d.k / d.group_size) * sb, per_unit * sb, per_unit * sb);
    sec(2, static_cast<const uint8_t *>(d.biases_dev), (d.k / d.group_size) * sb, per_unit * sb, per_unit * sb);
  }
  int off = 0;
  for (int i = 0; i < pl->nsec; ++i) {
    pl->src[i].sec_off = pl->sec_off[i] = off;
    pl->sec_bytes[i] = pl->src[i].field_bytes;
    off += kRowPanel * pl->src[i].field_bytes;  // a multiple of 256 bytes
  }
  pl->tile_bytes = off;
}

// Fixes grid, stage ring and scratch for one weight: two CTAs per SM, 128-row panels, kc units
// per stage.
bool make_row_plan(const ishi_ctx *ctx, const ishi_weight_desc &d, RowPlan *pl) {
  describe_sections(d, pl);
  pl->units = (int)(d.k / 256);
  pl->P = (int)((d.n + kRowPanel - 1) / kRowPanel);
  pl->grid = 2 * ctx->sm_count;
  const RowOps *rops = row_ops(format_of(d));
  if (!rops) return false;
  pl->table_bytes = rops->table_bytes;
  pl->tiles_bytes = (size_t)pl->P * pl->units * pl->tile_bytes;
  const size_t half_sm = (size_t)(std::min(kSmemPerSm, ctx->smem_optin) - 4096) / 2;
  const size_t fixed = 128 + (size_t)pl->table_bytes;
  for (pl->kc = pl->units >= 2 ? 2 : 1; pl->kc >= 1; --pl->kc) {
    pl->x_off = pl->kc * pl->tile_bytes;
    pl->bmin_off = pl->x_off + pl->kc * 4096;
    pl->xs_off = pl->bmin_off + pl->kc * 512;
    pl->stage_bytes = pl->xs_off + pl->kc * 256;
    if (fixed + 2 * (size_t)pl->stage_bytes <= half_sm) break;
  }
  if (pl->kc < 1) return false;
  int nst = 4;
  for (; nst >= 2; --nst) {
    pl->smem = fixed + (size_t)nst * pl->stage_bytes;
    if (pl->smem <= half_sm) break;
  }
  pl->nstages = nst;
  const long long Q = (long long)pl->P * pl->units;
  const int dense_slots = (pl->grid + pl->P - 1) / pl->P + 1;
  pl->SL = Q >= pl->grid ? dense_slots : std::max(pl->units, dense_slots);
  pl->scratch_floats = (size_t)pl->P * pl->SL * 8 * kRowPanel;
  pl->counters = (size_t)pl->P * 4;
  pl->ok = true;
  return true;
}

// st: the stream of the call the workspace is for; fresh counters are cleared on it, so the
// clearing is ordered before the call's kernels whatever kind of stream it is.
ishi_status ensure_workspace(ishi_ctx *ctx, Workspace *ws, size_t floats, size_t counters, size_t tiles,
                             cudaStream_t st) {
  if (floats > ws->scratch_floats) {
    if (ws->scratch) cudaFree(ws->scratch);
    ws->scratch = nullptr;
    ws->scratch_floats = 0;
    ISHI_CUDA(ctx, cudaMalloc(&ws->scratch, floats * sizeof(float)));
    ws->scratch_floats = floats;
  }
  if (counters > ws->n_counters) {
    if (ws->counters) cudaFree(ws->counters);
    ws->counters = nullptr;
    ws->n_counters = 0;
    ISHI_CUDA(ctx, cudaMalloc(&ws->counters, counters * sizeof(unsigned int)));
    ISHI_CUDA(ctx, cudaMemsetAsync(ws->counters, 0, counters * sizeof(unsigned int), st));
    ws->n_counters = counters;
    ws->epoch = ctx->timeout_epoch;
  }
  if (tiles > ws->tiles_bytes) {
    if (ws->tiles) cudaFree(ws->tiles);
    ws->tiles = nullptr;
    ws->tiles_bytes = 0;
    ISHI_CUDA(ctx, cudaMalloc(&ws->tiles, tiles));
    ws->tiles_bytes = tiles;
  }
  return ISHI_OK;
}

void free_workspace(Workspace *ws) {
  if (ws->scratch) cudaFree(ws->scratch);
  if (ws->counters) cudaFree(ws->counters);
  if (ws->tiles) cudaFree(ws->tiles);
  *ws = Workspace();
}

ishi_status tile_weight(ishi_ctx *ctx, const RowPlan &pl, long long n, uint8_t *dst, cudaStream_t st) {
  const long long triples = (long long)pl.P * pl.units * kRowPanel;
  const int grid = (int)std::min<long long>((triples + 255) / 256, (long long)ctx->sm_count * 16);
  prepare_tiles_kernel<<<grid, 256, 0, st>>>(pl.src[0], pl.src[1], pl.src[2], pl.src[3], pl.nsec, n, pl.units,
                                             pl.tile_bytes, dst);
  ISHI_CUDA(ctx, cudaGetLastError());
  return ISHI_OK;
}

// Raises a kernel family's shared-memory limit once per device.
ishi_status configure_once(ishi_ctx *ctx, const void *key, cudaError_t (*configure)(int), int max_smem) {
  static std::map<std::pair<const void *, int>, bool> done;
  static std::mutex once;
  std::lock_guard<std::mutex> g(once);
  bool &flag = done[std::make_pair(key, ctx->device)];
  if (!flag) {
    ISHI_CUDA(ctx, configure(max_smem));
    flag = true;
  }
  return ISHI_OK;
}

ishi_status launch_row(ishi_ctx *ctx, int fmt, const RowPlan &pl, const RowArgs &args, cudaStream_t st) {
  const RowOps *ops = row_ops(fmt);
  if (!ops) return fail(ctx, ISHI_E_UNSUPPORTED, "no kernel for format %d", fmt);
  ishi_status s = configure_once(ctx, ops, ops->configure, (std::min(kSmemPerSm, ctx->smem_optin) - 4096) / 2);
  if (s != ISHI_OK) return s;
  ISHI_CUDA(ctx, ops->launch(args.M, pl.grid, pl.smem, args, st));
  return ISHI_OK;
}

// One launch: x [rows <= 8, k] against the tiled weight.
ishi_status run_row(ishi_ctx *ctx, const RowPlan &pl, const Workspace &ws, int fmt, const ishi_weight_desc &d,
                    const void *x, int rows, void *y, long long ldy, int flags, cudaStream_t st) {
  RowArgs a;
  memset(&a, 0, sizeof(a));
  a.tiles = ws.tiles;
  a.tile_bytes = pl.tile_bytes;
  for (int i = 0; i < 4; ++i) {
    a.sec_off[i] = pl.sec_off[i];
    a.sec_bytes[i] = pl.sec_bytes[i];
  }
  a.x = static_cast<const __half *>(x);
  a.y = static_cast<__half *>(y);
  a.ldy = ldy;
  a.out_transposed = (flags & ISHI_OUT_TRANSPOSED) ? 1 : 0;
  if (ws.counters && ws.epoch != ctx->timeout_epoch) {
    // a launch on this context timed out since these counters were last zero
    ISHI_CUDA(ctx, cudaMemsetAsync(ws.counters, 0, ws.n_counters * sizeof(unsigned int), st));
    ws.epoch = ctx->timeout_epoch;
  }
  a.scratch = ws.scratch;
  a.counters = ws.counters;
  a.err = ctx->err_dev;
  a.M = rows;
  a.N = (int)d.n;
  a.K = (int)d.k;
  a.units = pl.units;
  a.P = pl.P;
  a.SL = pl.SL;
  a.kc = pl.kc;
  a.nstages = pl.nstages;
  a.x_off = pl.x_off;
  a.bmin_off = pl.bmin_off;
  a.xs_off = pl.xs_off;
  a.stage_bytes = pl.stage_bytes;
  a.group_size = d.group_size;
  a.scale_dtype = d.scale_dtype;
  a.bits = d.bits;
  return launch_row(ctx, fmt, pl, a, st);
}

// rows 1...16: one launch for up to eight rows, two for more (the weight then streams twice).
ishi_status run_rows(ishi_ctx *ctx, const RowPlan &pl, const Workspace &ws, int fmt, const ishi_weight_desc &d,
                     const void *x, int rows, void *y, long long ldy, int flags, cudaStream_t st) {
  for (int r0 = 0; r0 < rows; r0 += 8) {
    const int nr = std::min(8, rows - r0);
    const __half *xs = static_cast<const __half *>(x) + (long long)r0 * d.k;
    __half *ys = static_cast<__half *>(y) + ((flags & ISHI_OUT_TRANSPOSED) ? (long long)r0 : (long long)r0 * ldy);
    ishi_status s = run_row(ctx, pl, ws, fmt, d, xs, nr, ys, ldy, flags, st);
    if (s != ISHI_OK) return s;
  }
  return ISHI_OK;
}

// ---- warp-level kernel: plan, tiling, launch ------------------------------------------------------

// The fragment decoder that serves a weight, or null (the tcgen05 kernel then takes it, as it does
// when no plan of the warp-level kernel fits shared memory: very wide inputs).
const FragOps *frag_ops_for(const ishi_weight_desc &d) {
  // ISHI_KERNEL=tcgen05: every weight goes to the tcgen05 kernel (to compare the two kernels on one format)
  const char *which = getenv("ISHI_KERNEL");
  if (which && strcmp(which, "tcgen05") == 0) return nullptr;
  if (d.kind == ISHI_KIND_GGML) {
    if (d.ggml_type == ISHI_GGML_Q4_K) return frag_ops_q4k();
    if (d.ggml_type == ISHI_GGML_Q6_K) return frag_ops_q6k();
    if (d.ggml_type == ISHI_GGML_IQ2_XS) return frag_ops_iq2xs();
    // ISHI_DENSE_DECODER=1: the eight other types through the dense decoder instead of their own
    // fragment decoders (to compare the two, and to keep that path exercised)
    if (!getenv("ISHI_DENSE_DECODER")) {
      if (d.ggml_type == ISHI_GGML_IQ4_XS) return frag_ops_iq4xs();
      if (d.ggml_type == ISHI_GGML_IQ2_XXS) return frag_ops_iq2xxs();
      if (d.ggml_type == ISHI_GGML_IQ2_S) return frag_ops_iq2s();
      if (d.ggml_type == ISHI_GGML_IQ3_XXS) return frag_ops_iq3xxs();
      if (d.ggml_type == ISHI_GGML_IQ3_S) return frag_ops_iq3s();
      if (d.ggml_type == ISHI_GGML_Q2_K) return frag_ops_q2k();
      if (d.ggml_type == ISHI_GGML_IQ1_S) return frag_ops_iq1s();
      if (d.ggml_type == ISHI_GGML_IQ1_M) return frag_ops_iq1m();
    }
    if (const FragOps *ops = frag_ops_ggml_a(d.ggml_type)) return ops;
    return frag_ops_ggml_b(d.ggml_type);  // the other block types, through the dense decoder
  }
  if (d.scale_dtype != ISHI_DT_F16 && d.scale_dtype != ISHI_DT_BF16) return nullptr;
  const bool bf16 = d.scale_dtype == ISHI_DT_BF16;
  if (d.bits == 4) return frag_ops_affine4(d.group_size, bf16);
  if (d.bits == 2) return frag_ops_affine2(d.group_size, bf16);
  return nullptr;
}

// how many clusters of s CTAs with this much shared memory the device runs at once
int max_frag_clusters(ishi_ctx *ctx, const FragOps *ops, int s, int warps, size_t smem) {
  static std::map<std::tuple<int, const void *, int, int, size_t>, int> cache;
  static std::mutex lock;
  std::lock_guard<std::mutex> g(lock);
  const auto key = std::make_tuple(ctx->device, (const void *)ops, s, warps, smem);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  const int n = ops->max_clusters(s, warps, smem, ctx->sm_count);
  cache[key] = n;
  return n;
}

// Picks the K split S (= cluster size), the warps per panel and the panels a CTA works on in
// parallel. The estimate counts tile times on the longest warp (panels of the fullest cluster x
// units per warp), stretched where the warps outnumber what the issue slots sustain.
bool make_frag_plan(ishi_ctx *ctx, const ishi_weight_desc &d, FragPlan *pl, std::vector<FragPlan> *all = nullptr) {
  const FragOps *ops = frag_ops_for(d);
  if (!ops) return false;
  const size_t budget = (size_t)std::min(kSmemPerSm, ctx->smem_optin) - 1024;
  if (configure_once(ctx, ops, ops->configure, (int)budget) != ISHI_OK) return false;
  const int xbytes = ops->x_bytes;
  FragPlan best;
  const int tile_bytes = ops->tile_bytes;
  const int units = (int)(d.k / 256);
  const int P = (int)((d.n + kFragRows - 1) / kFragRows);
  // the kernel divides by multiplication, exact while (clusters + 1) * P < 2^32 / clusters
  if ((long long)P * (ctx->sm_count + 1) * ctx->sm_count >= (1ll << 32)) return false;
  const char *force = getenv("ISHI_FRAG_PLAN");  // "S,per,PP[,ring]" for tuning runs
  int fs = 0, fper = 0, fpp = 0, fring = 0;
  if (force) sscanf(force, "%d,%d,%d,%d", &fs, &fper, &fpp, &fring);
  for (int s = 1; s <= kFragMaxSplit && s <= units; ++s) {
    if (fs && s != fs) continue;
    const int umax = (units + s - 1) / s;
    const int per_min = (umax + kFragMaxWarps - 1) / kFragMaxWarps;
    // units per warp: a few around the fewest that fit the warps, and the whole range and half of
    // it in one warp (no or little adding up between the warps of a panel)
    const int per_hi = std::min(per_min + 2, kFragGroup);
    for (int per = per_min; per <= umax; ++per) {
      if (fper ? per != fper : (per > per_hi && per != umax && per != (umax + 1) / 2)) continue;
      const int wu = (umax + per - 1) / per;
      for (int pp = 1; pp <= kFragMaxPanels && wu * pp <= kFragMaxWarps; ++pp) {
        if (fpp && pp != fpp) continue;
        FragPlan c;
        c.ops = ops;
        c.units = units;
        c.P = P;
        c.S = s;
        c.tile_bytes = tile_bytes;
        c.umax = umax;
        c.Wu = wu;
        c.PP = pp;
        const int w = wu * pp;
        // the deepest tile ring that fits, then the larger inbox generation
        bool fits = false;
        for (int ring = fring ? fring : 3; ring >= (fring ? fring : 2) && !fits; --ring)
          for (int gen = 2; gen >= 1 && !fits; --gen) {
            const size_t need = frag_smem_bytes((size_t)umax * xbytes + ops->x_extra, w, pp, gen, s, tile_bytes, ring);
            if (need <= budget) {
              fits = true;
              c.ring = ring, c.G = gen, c.smem = need;
            }
          }
        if (!fits) continue;
        // one CTA per SM: two would stage the activations twice and split the issue slots
        c.NC = std::min(std::min(max_frag_clusters(ctx, ops, s, w, c.smem), ctx->sm_count / s), P);
        if (c.NC < 1) continue;
        // Estimate in microseconds, fitted to measurements on the 27B shapes: an SM passes about
        // 13 tiles per microsecond when enough warps are busy; one warp alone needs about a
        // microsecond per tile; every panel of a lane costs a reduction over its wu warps.
        const int panels = (P + c.NC - 1) / c.NC;
        const int rounds = (panels + pp - 1) / pp;  // panels one warp walks
        const double throughput = 0.075 * panels * umax * std::max(1.0, 14.0 / w);
        const double longest = 1.0 * rounds * per;
        c.cost = std::max(throughput, longest) + rounds * (0.05 * wu + (s > 1 ? 0.05 : 0.0)) + 0.02 * umax;
        c.ok = true;
        c.tiles_bytes = (size_t)P * units * tile_bytes;
        if (all) all->push_back(c);
        if (!best.ok || c.cost < best.cost) best = c;
      }
    }
  }
  if (!best.ok) return false;
  best.tiles_bytes = (size_t)P * units * tile_bytes;
  if (getenv("ISHI_DEBUG_PLAN"))
    fprintf(stderr, "ishi plan n=%lld k=%lld: split %d, clusters %d, warps %d x %d, generation %d, ring %d, smem %zu\n",
            (long long)d.n, (long long)d.k, best.S, best.NC, best.Wu, best.PP, best.G, best.ring, best.smem);
  *pl = best;
  return true;
}

ishi_status tile_weight_frag(ishi_ctx *ctx, const FragPlan &pl, const ishi_weight_desc *parts, int count, long long n_total,
                             uint8_t *dst, cudaStream_t st, bool pair_rows = false) {
  FragSrc src;
  memset(&src, 0, sizeof(src));
  src.pair_rows = pair_rows ? 1 : 0;
  const ishi_weight_desc &d = parts[0];
  src.N = n_total;
  src.segments = count;
  long long row = 0;
  for (int i = 0; i < count; ++i) {
    src.w[i] = static_cast<const uint8_t *>(parts[i].weight_dev);
    src.scales[i] = static_cast<const uint8_t *>(parts[i].scales_dev);
    src.biases[i] = static_cast<const uint8_t *>(parts[i].biases_dev);
    src.first_row[i] = row;
    row += parts[i].n;
  }
  for (int i = count; i <= kFragMaxSegments; ++i) src.first_row[i] = row;
  if (d.kind == ISHI_KIND_GGML) {
    src.w_row_bytes = (long long)(d.k / 256) * type_size(d.ggml_type);
  } else {
    src.w_row_bytes = (long long)d.k * d.bits / 8;
    src.group_size = d.group_size;
    src.scale_bytes = 2;
    src.s_row_bytes = (long long)(d.k / d.group_size) * 2;
  }
  const long long total = (long long)pl.P * pl.units * (pl.tile_bytes / 2);
  const int grid = (int)std::min<long long>((total + 255) / 256, (long long)ctx->sm_count * 32);
  ISHI_CUDA(ctx, pl.ops->prepare(src, pl.units, dst, grid, st));
  return ISHI_OK;
}

#ifdef ISHI_TRACE
unsigned long long *g_trace = nullptr;  // diagnostic builds: where the kernels stamp their phases
#endif

// where a sharded product stores its rows (see ishi_exchange_apply)
struct PeerOut {
  int world, rank;
  __half *y[kFragMaxPeers];
  unsigned *flags[kFragMaxPeers];
  unsigned *local_flags, *done, *launch_no;
  int wait_previous;
  long long row_offset;
};

// Does a single row go to the CUDA-core kernel? ISHI_ROUTE_GEMV: yes; ISHI_ROUTE_MMA: no; AUTO: when
// the crossover is above one row. The built-in crossover is 1 (the tensor-core kernel is the faster
// one on B200 at every row count, measured per shape in the benchmark's side table).
bool single_row_on_cuda_cores(const ishi_ctx *ctx) {
  if (ctx->route == ISHI_ROUTE_GEMV) return true;
  if (ctx->route == ISHI_ROUTE_MMA) return false;
  return ctx->crossover_rows > 1;
}

// rows 1...16 through the warp-level kernel; gemv picks the CUDA-core variant for a single row
ishi_status run_frag(ishi_ctx *ctx, const FragPlan &pl, const Workspace &ws, const ishi_weight_desc &d, const void *x,
                     int rows, void *y, long long ldy, int flags, bool gemv, bool early, bool rotate, cudaStream_t st,
                     const PeerOut *peers = nullptr, bool gated = false) {
  for (int r0 = 0; r0 < rows; r0 += 8) {
    FragArgs a;
    memset(&a, 0, sizeof(a));
    a.tiles = ws.tiles;
    a.x = static_cast<const __half *>(x) + (long long)r0 * d.k;
    a.y = static_cast<__half *>(y) + ((flags & ISHI_OUT_TRANSPOSED) ? (long long)r0 : (long long)r0 * ldy);
    a.ldy = ldy;
    a.out_transposed = (flags & ISHI_OUT_TRANSPOSED) ? 1 : 0;
    a.M = std::min(8, rows - r0);
    a.N = (int)d.n;
    a.K = (int)d.k;
    a.units = pl.units;
    a.S = pl.S;
    a.P = pl.P;
    a.NC = pl.NC;
    a.Wu = pl.Wu;
    a.PP = pl.PP;
    a.G = pl.G;
    a.ring = pl.ring;
    a.inv_s = frag_inverse(pl.S);
    a.inv_nc = frag_inverse(pl.NC);
    a.inv_wu = frag_inverse(pl.Wu);
    a.inv_pp = frag_inverse(pl.PP);
    a.umax = pl.umax;
    a.group_size = d.group_size;
    a.scale_dtype = d.scale_dtype;
    a.err = ctx->err_dev;
    a.rot_block = rotate ? d.hadamard_block : 0;
    a.rot_signs = rotate ? static_cast<const float *>(d.signs_dev) : nullptr;
    a.swiglu = gated ? 1 : 0;
#ifdef ISHI_TRACE
    a.trace = g_trace;
#endif
    if (peers) {
      a.world = peers->world;
      a.rank = peers->rank;
      a.peer_ld = rows > 8 ? 16 : 8;  // the second piece of eight rows lies beside the first
      for (int q = 0; q < peers->world; ++q) {
        a.peer_y[q] = peers->y[q] + r0;
        a.peer_flags[q] = peers->flags[q];
      }
      a.local_flags = peers->local_flags;
      a.done = peers->done;
      a.launch_no = peers->launch_no;
      a.wait_previous = peers->wait_previous;
      a.row_offset = peers->row_offset;
    }
    FragLaunch l;
    l.clusters = pl.NC;
    l.split = pl.S;
    l.warps = pl.Wu * pl.PP;
    l.smem = pl.smem;
    l.mode = (gemv && rows == 1) ? 1 : 0;
    l.early = early;
    l.stream = st;
    ISHI_CUDA(ctx, pl.ops->launch(l, a));
  }
  return ISHI_OK;
}

ishi_status check_io(ishi_ctx *ctx, const void *x, int rows, const void *y, int max_rows) {
  if (!x || !y) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (!aligned16(x)) return fail(ctx, ISHI_E_INVALID, "x must be 16-byte aligned");
  if (rows < 1 || rows > max_rows) return fail(ctx, ISHI_E_SHAPE, "rows %d outside 1...%d", rows, max_rows);
  return ISHI_OK;
}

// Kernel-level product on a caller's raw weight: re-tiles it into the context's buffer, then runs.
ishi_status raw_product(ishi_ctx *ctx, const ishi_weight_desc &d, const void *x, int rows, void *y, bool gemv,
                        cudaStream_t st) {
  int64_t wb = 0;
  ishi_status s = check_desc(ctx, d, &wb);
  if (s != ISHI_OK) return s;
  std::lock_guard<std::mutex> g(ctx->lock);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  FragPlan fp;
  if (make_frag_plan(ctx, d, &fp)) {
    s = ensure_workspace(ctx, &ctx->ws, 0, 0, fp.tiles_bytes, st);
    if (s != ISHI_OK) return s;
    s = tile_weight_frag(ctx, fp, &d, 1, d.n, ctx->ws.tiles, st);
    if (s != ISHI_OK) return s;
    return run_frag(ctx, fp, ctx->ws, d, x, rows, y, d.n, 0, gemv || single_row_on_cuda_cores(ctx), false, false, st);
  }
  RowPlan pl;
  if (!make_row_plan(ctx, d, &pl)) {
    if (d.kind == ISHI_KIND_GGML && !row_ops(format_of(d))) {
      // a block format without a streaming kernel: one warp per output row on the caller's blocks
      ISHI_CUDA(ctx, launch_ggml_rowdot(d.ggml_type, static_cast<const uint8_t *>(d.weight_dev), d.n, d.k,
                                        static_cast<const __half *>(x), rows, static_cast<__half *>(y), d.n, 0,
                                        ctx->sm_count, st));
      return ISHI_OK;
    }
    return fail(ctx, ISHI_E_SHAPE, "no launch plan fits shared memory");
  }
  s = ensure_workspace(ctx, &ctx->ws, pl.scratch_floats, pl.counters, pl.tiles_bytes, st);
  if (s != ISHI_OK) return s;
  s = tile_weight(ctx, pl, d.n, ctx->ws.tiles, st);
  if (s != ISHI_OK) return s;
  return run_rows(ctx, pl, ctx->ws, format_of(d), d, x, rows, y, d.n, 0, st);
}

ishi_status ggml_raw(ishi_ctx *ctx, const void *x, int rows, const void *blocks, int64_t blocks_bytes, int type,
                     int64_t n, int64_t k, void *y, bool gemv, void *stream) {
  if (!ctx) return ISHI_E_INVALID;
  ishi_status s = check_io(ctx, x, rows, y, 16);
  if (s != ISHI_OK) return s;
  ishi_weight_desc d;
  memset(&d, 0, sizeof(d));
  d.kind = ISHI_KIND_GGML;
  d.ggml_type = type;
  d.n = n;
  d.k = k;
  d.weight_dev = blocks;
  d.weight_bytes = blocks_bytes;
  return raw_product(ctx, d, x, rows, y, gemv, static_cast<cudaStream_t>(stream));
}

// The warp-level kernel rotates x while it stages it when a block fits one 256-wide unit: the
// staging of the affine packs does (the reference's rotated packs are affine, Hadamard.swift:51-86);
// the GGUF decoders' staging does not, their input is rotated by the stand-alone kernel first.
bool rotates_in_kernel(const ishi_projection *p) {
  const int b = p->d.hadamard_block;
  return p->frag.ok && p->d.kind == ISHI_KIND_AFFINE && b >= 8 && b <= 256 && (b & (b - 1)) == 0;
}

// rotate: x is unrotated and the projection's rotation is applied inside the product kernel
ishi_status projection_matmul(ishi_projection *p, const void *x, int rows, void *y, int64_t ldy, int flags,
                              bool rotate, cudaStream_t st) {
  ishi_ctx *ctx = p->ctx;
  ishi_status s = check_io(ctx, x, rows, y, 16);
  if (s != ISHI_OK) return s;
  const int64_t need_ld = (flags & ISHI_OUT_TRANSPOSED) ? rows : out_rows(p);
  if (ldy < need_ld) return fail(ctx, ISHI_E_SHAPE, "ldy %lld shorter than %lld", (long long)ldy, (long long)need_ld);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  if (p->frag.ok)
    return run_frag(ctx, p->frag, p->ws, p->d, x, rows, y, ldy, flags, single_row_on_cuda_cores(ctx),
                    getenv("ISHI_NO_EARLY_LAUNCH") == nullptr, rotate, st, nullptr, p->gated);
  if (p->generic) {
    if (rotate) return fail(ctx, ISHI_E_INVALID, "in-kernel rotation asked of a kernel that has none");
    ISHI_CUDA(ctx, launch_ggml_rowdot(p->d.ggml_type, p->ws.tiles, p->d.n, p->d.k, static_cast<const __half *>(x), rows,
                                      static_cast<__half *>(y), ldy, (flags & ISHI_OUT_TRANSPOSED) ? 1 : 0, ctx->sm_count, st));
    return ISHI_OK;
  }
  if (rotate) return fail(ctx, ISHI_E_INVALID, "in-kernel rotation asked of a kernel that has none");
  return run_rows(ctx, p->plan, p->ws, p->fmt, p->d, x, rows, y, ldy, flags, st);
}

}  // namespace

// ---------------------------------------------------------------------------------------------

extern "C" {

#ifdef ISHI_TRACE
void ishi_debug_set_trace(void *dev) { g_trace = static_cast<unsigned long long *>(dev); }
#endif

const char *ishi_status_string(ishi_status s) {
  switch (s) {
    case ISHI_OK: return "ok";
    case ISHI_E_INVALID: return "invalid argument";
    case ISHI_E_SHAPE: return "shape outside the supported range";
    case ISHI_E_UNSUPPORTED: return "unsupported format";
    case ISHI_E_CUDA: return "CUDA error";
    case ISHI_E_TIMEOUT: return "device-side wait timed out";
    case ISHI_E_NOMEM: return "out of memory";
    case ISHI_E_TOO_LARGE: return "larger than the built-in scratch of the no-allocation entry point";
    case ISHI_E_NCCL: return "NCCL error";
    default: return "unknown status";
  }
}

const char *ishi_last_error(const ishi_ctx *ctx) { return ctx ? ctx->last_error : "null context"; }

ishi_status ishi_ctx_create(int device, ishi_ctx **out) {
  if (!out) return ISHI_E_INVALID;
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return ISHI_E_CUDA;
  ishi_ctx *ctx = new (std::nothrow) ishi_ctx();
  if (!ctx) return ISHI_E_NOMEM;
  ctx->device = device;
  cudaError_t e = cudaSetDevice(device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&ctx->smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
  int major = 0;
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (e == cudaSuccess && major != 10) {
    delete ctx;
    return ISHI_E_UNSUPPORTED;  // the kernels are built for sm_100a only
  }
  if (e == cudaSuccess) e = cudaHostAlloc(&ctx->err_host, sizeof(int), cudaHostAllocMapped);
  if (e == cudaSuccess) {
    *ctx->err_host = 0;
    e = cudaHostGetDevicePointer(&ctx->err_dev, ctx->err_host, 0);
  }
  if (e != cudaSuccess) {
    if (ctx->err_host) cudaFreeHost(ctx->err_host);
    delete ctx;
    return ISHI_E_CUDA;
  }
  *out = ctx;
  return ISHI_OK;
}

void ishi_ctx_destroy(ishi_ctx *ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  free_workspace(&ctx->ws);
  if (ctx->err_host) cudaFreeHost(ctx->err_host);
  if (ctx->pin_x) cudaFreeHost(ctx->pin_x);
  if (ctx->pin_y) cudaFreeHost(ctx->pin_y);
  if (ctx->dev_x) cudaFree(ctx->dev_x);
  if (ctx->dev_y) cudaFree(ctx->dev_y);
  if (ctx->exl3_x) cudaFree(ctx->exl3_x);
  if (ctx->exl3_y) cudaFree(ctx->exl3_y);
  for (cudaEvent_t e : ctx->ev_in) cudaEventDestroy(e);
  for (cudaEvent_t e : ctx->ev_done) cudaEventDestroy(e);
  if (ctx->ev_begin) cudaEventDestroy(ctx->ev_begin);
  if (ctx->ev_end) cudaEventDestroy(ctx->ev_end);
  if (ctx->copy_in) cudaStreamDestroy(ctx->copy_in);
  if (ctx->copy_out) cudaStreamDestroy(ctx->copy_out);
  delete ctx;
}

ishi_status ishi_ctx_poll(ishi_ctx *ctx) {
  if (!ctx) return ISHI_E_INVALID;
  volatile int *flag = ctx->err_host;
  if (*flag != 0) {
    *flag = 0;
    ++ctx->timeout_epoch;  // CTAs that gave up skipped their arrivals: run_row clears the counters before their next use
    return fail(ctx, ISHI_E_TIMEOUT, "a kernel's bounded wait gave up; outputs of that launch are invalid");
  }
  return ISHI_OK;
}

ishi_status ishi_ctx_set_route(ishi_ctx *ctx, int route, int crossover_rows) {
  if (!ctx) return ISHI_E_INVALID;
  if (route < ISHI_ROUTE_AUTO || route > ISHI_ROUTE_MMA || crossover_rows < 0 || crossover_rows > 17)
    return fail(ctx, ISHI_E_INVALID, "route %d / crossover %d out of range", route, crossover_rows);
  ctx->route = route;
  ctx->crossover_rows = crossover_rows;
  return ISHI_OK;
}

int ishi_reference_minimum_rows(int64_t bytes) {
  if (bytes >= 100000000) return 2;
  if (bytes >= 10000000) return 3;
  if (bytes >= 5000000) return 4;
  return 6;
}

int ishi_ggml_block_size(int t) { return type_size(t) ? 256 : 0; }
int ishi_ggml_type_size(int t) { return type_size(t); }

ishi_status ishi_ggml_dequantize(ishi_ctx *ctx, int type, const void *blocks, int64_t n_blocks, void *out,
                                 int out_dtype, void *stream) {
  if (!ctx) return ISHI_E_INVALID;
  if (!blocks || !out) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (type_size(type) == 0) return fail(ctx, ISHI_E_UNSUPPORTED, "GGML type %d has no decoder here", type);
  if (n_blocks < 0) return fail(ctx, ISHI_E_SHAPE, "negative block count");
  if (n_blocks == 0) return ISHI_OK;
  if (out_dtype < ISHI_DT_F16 || out_dtype > ISHI_DT_F32) return fail(ctx, ISHI_E_INVALID, "bad output dtype %d", out_dtype);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  ISHI_CUDA(ctx, launch_ggml_dequantize(type, static_cast<const uint8_t *>(blocks), n_blocks, out, out_dtype, ctx->sm_count,
                                        static_cast<cudaStream_t>(stream)));
  return ISHI_OK;
}

ishi_status ishi_ggml_gather(ishi_ctx *ctx, const int32_t *ids, int64_t count, const void *blocks, int64_t blocks_bytes,
                             int type, int64_t table_rows, int64_t k, void *out, int out_dtype, void *stream) {
  if (!ctx) return ISHI_E_INVALID;
  if (!ids || !blocks || !out) return fail(ctx, ISHI_E_INVALID, "null pointer");
  const int ts = type_size(type);
  if (ts == 0) return fail(ctx, ISHI_E_UNSUPPORTED, "GGML type %d has no decoder here", type);
  if (out_dtype < ISHI_DT_F16 || out_dtype > ISHI_DT_F32) return fail(ctx, ISHI_E_INVALID, "bad output dtype %d", out_dtype);
  if (count < 0 || table_rows <= 0 || k <= 0 || k % 256 != 0)
    return fail(ctx, ISHI_E_SHAPE, "input width %lld is not a whole number of blocks", (long long)k);
  if (blocks_bytes < table_rows * (k / 256) * ts)
    return fail(ctx, ISHI_E_SHAPE, "table buffer holds %lld bytes, shape needs %lld", (long long)blocks_bytes,
                (long long)(table_rows * (k / 256) * ts));
  if (count == 0) return ISHI_OK;
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  ISHI_CUDA(ctx, launch_ggml_gather(type, ids, count, static_cast<const uint8_t *>(blocks), table_rows, k, out, out_dtype,
                                    ctx->sm_count, static_cast<cudaStream_t>(stream)));
  return ISHI_OK;
}

ishi_status ishi_affine_dequantize(ishi_ctx *ctx, const void *w, const void *scales, const void *biases,
                                   int scale_dtype, int group_size, int bits, int64_t n, int64_t k, float *out,
                                   void *stream) {
  if (!ctx) return ISHI_E_INVALID;
  if (!w || !scales || !biases || !out) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (bits < 2 || bits > 8) return fail(ctx, ISHI_E_SHAPE, "bits %d outside 2...8", bits);
  if (scale_dtype < ISHI_DT_F16 || scale_dtype > ISHI_DT_F32) return fail(ctx, ISHI_E_INVALID, "bad scale dtype");
  if (group_size <= 0 || k <= 0 || n <= 0 || k % group_size != 0 || (k * bits) % 32 != 0)
    return fail(ctx, ISHI_E_SHAPE, "k %lld does not fit groups of %d at %d bits", (long long)k, group_size, bits);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  const long long total = n * k;
  const int grid = (int)std::min<long long>((total + 255) / 256, (long long)ctx->sm_count * 32);
  affine_dequantize_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t *>(w), scales, biases, scale_dtype, group_size, bits, n, k, out);
  ISHI_CUDA(ctx, cudaGetLastError());
  return ISHI_OK;
}

ishi_status ishi_hadamard_rotate(ishi_ctx *ctx, const void *x, int64_t rows, int64_t width, int block,
                                 const float *signs, void *y, void *stream) {
  if (!ctx) return ISHI_E_INVALID;
  if (!x || !y) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (block <= 0 || (block & (block - 1)) != 0 || block > 8192)
    return fail(ctx, ISHI_E_SHAPE, "Hadamard block %d is not a power of two up to 8192", block);
  if (rows <= 0 || width <= 0 || width % block != 0)
    return fail(ctx, ISHI_E_SHAPE, "Hadamard block %d does not divide activation width %lld", block, (long long)width);
  const long long grid = rows * (width / block);
  if (grid > 0x7fffffffll) return fail(ctx, ISHI_E_SHAPE, "too many blocks");
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  const int threads = std::max(32, std::min(256, block / 2));
  hadamard_rotate_kernel<<<(int)grid, threads, block * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half *>(x), width, block, signs, static_cast<__half *>(y));
  ISHI_CUDA(ctx, cudaGetLastError());
  return ISHI_OK;
}

ishi_status ishi_ggml_matmul_few(ishi_ctx *ctx, const void *x, int rows, const void *blocks, int64_t blocks_bytes,
                                 int type, int64_t n, int64_t k, void *y, void *stream) {
  return ggml_raw(ctx, x, rows, blocks, blocks_bytes, type, n, k, y, false, stream);
}

ishi_status ishi_ggml_matvec(ishi_ctx *ctx, const void *x, int rows, const void *blocks, int64_t blocks_bytes,
                             int type, int64_t n, int64_t k, void *y, void *stream) {
  // a single row runs on CUDA cores where the format has that kernel; more rows, or other
  // formats, take the tensor-core kernel
  return ggml_raw(ctx, x, rows, blocks, blocks_bytes, type, n, k, y, true, stream);
}

ishi_status ishi_verify_matmul(ishi_ctx *ctx, const void *x, int rows, const void *w, const void *scales,
                               const void *biases, int scale_dtype, int group_size, int bits, int64_t n, int64_t k,
                               int route, void *y, void *stream) {
  if (!ctx) return ISHI_E_INVALID;
  (void)route;
  ishi_status s = check_io(ctx, x, rows, y, 16);
  if (s != ISHI_OK) return s;
  ishi_weight_desc d;
  memset(&d, 0, sizeof(d));
  d.kind = ISHI_KIND_AFFINE;
  d.bits = bits;
  d.group_size = group_size;
  d.scale_dtype = scale_dtype;
  d.n = n;
  d.k = k;
  d.weight_dev = w;
  d.weight_bytes = (bits >= 2 && bits <= 8 && n > 0 && k > 0) ? n * k * bits / 8 : 0;
  d.scales_dev = scales;
  d.biases_dev = biases;
  return raw_product(ctx, d, x, rows, y, route == ISHI_ROUTE_GEMV, static_cast<cudaStream_t>(stream));
}

// ---- projection: the PackedLinear counterpart ---------------------------------------------------

// The tile layout does not depend on the launch plan, so the plan can be chosen by measurement:
// the planner's best candidates run a few times on the projection's own tiles (activations of
// zeros, eight rows) and the fastest stays. The estimate alone is within ~15 % of the best plan.
static void tune_frag_plan(ishi_ctx *ctx, ishi_projection *p, std::vector<FragPlan> *candidates) {
  constexpr size_t kTuned = 24;
  constexpr int kLaunches = 4;
  if (candidates->size() < 2) return;
  // a shape measured before on this context keeps its plan (all layers of a model then agree)
  const auto key = std::make_tuple((const void *)p->frag.ops, (long long)p->d.n, (long long)p->d.k);
  const auto known = ctx->tuned.find(key);
  if (known != ctx->tuned.end()) {
    for (const FragPlan &c : *candidates)
      if (c.S == known->second[0] && c.Wu == known->second[1] && c.PP == known->second[2] && c.ring == known->second[3]) {
        p->frag = c;
        return;
      }
  }
  std::sort(candidates->begin(), candidates->end(), [](const FragPlan &a, const FragPlan &b) { return a.cost < b.cost; });
  if (candidates->size() > kTuned) candidates->resize(kTuned);
  __half *x = nullptr, *y = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  bool ok = cudaMalloc(&x, (size_t)8 * p->d.k * sizeof(__half)) == cudaSuccess &&
            cudaMalloc(&y, (size_t)8 * p->d.n * sizeof(__half)) == cudaSuccess &&
            cudaMemset(x, 0, (size_t)8 * p->d.k * sizeof(__half)) == cudaSuccess && cudaEventCreate(&e0) == cudaSuccess &&
            cudaEventCreate(&e1) == cudaSuccess;
  // one timing: a warm-up launch, then `launches` back to back between two events
  auto time_plan = [&](const FragPlan &c, int launches, float *ms_per_launch) {
    bool fine = run_frag(ctx, c, p->ws, p->d, x, 8, y, p->d.n, 0, false, true, false, 0) == ISHI_OK;
    if (fine) fine = cudaEventRecord(e0, 0) == cudaSuccess;
    for (int r = 0; fine && r < launches; ++r) fine = run_frag(ctx, c, p->ws, p->d, x, 8, y, p->d.n, 0, false, true, false, 0) == ISHI_OK;
    if (fine) fine = cudaEventRecord(e1, 0) == cudaSuccess && cudaEventSynchronize(e1) == cudaSuccess;
    float ms = 0.f;
    if (fine) fine = cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess;
    *ms_per_launch = ms / launches;
    return fine;
  };
  // first pass over all candidates, then the best few again with more launches (the first pass
  // alone picks among near-equal plans by noise)
  constexpr size_t kFinalists = 4;
  std::vector<std::pair<float, const FragPlan *>> timed;
  for (size_t i = 0; ok && i < candidates->size(); ++i) {
    float ms = 0.f;
    ok = time_plan((*candidates)[i], kLaunches, &ms);
    if (ok) timed.push_back({ms, &(*candidates)[i]});
  }
  std::sort(timed.begin(), timed.end(), [](const auto &a, const auto &b) { return a.first < b.first; });
  float best_ms = 0.f;
  const FragPlan *best = nullptr;
  std::vector<std::pair<float, const FragPlan *>> finals;
  for (size_t i = 0; ok && i < timed.size() && i < kFinalists; ++i) {
    float ms = 0.f;
    ok = time_plan(*timed[i].second, 4 * kLaunches, &ms);
    if (ok) finals.push_back({ms, timed[i].second});
    if (ok && (!best || ms < best_ms)) best = timed[i].second, best_ms = ms;
  }
  // Near-equal finalists: the smaller cluster wins. The timing repeats one launch, where the SMs
  // fall free in the pattern the next launch's clusters need; between launches of different shapes
  // a large cluster waits longer for its SMs of one GPC, which this timing does not see (measured
  // on the benchmark's stack: 3 % per layer between K splits of 4 and 5 that time within 2 %).
  const char *tie_env = getenv("ISHI_TUNE_TIE");
  const float tie = tie_env ? (float)atof(tie_env) * 0.01f : 0.03f;
  if (ok && best)
    for (const auto &f : finals)
      if (f.first <= best_ms * (1.f + tie) && f.second->S < best->S) best = f.second;
  if (ok && best) {
    p->frag = *best;
    ctx->tuned[key] = {best->S, best->Wu, best->PP, best->ring};
    if (getenv("ISHI_DEBUG_PLAN"))
      fprintf(stderr, "ishi plan n=%lld k=%lld measured: split %d, warps %d x %d, ring %d: %.2f us\n", (long long)p->d.n,
              (long long)p->d.k, best->S, best->Wu, best->PP, best->ring, best_ms * 1e3f);
  } else {
    cudaGetLastError();  // keep the estimate's choice
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (x) cudaFree(x);
  if (y) cudaFree(y);
}

static ishi_status create_projection(ishi_ctx *ctx, const ishi_weight_desc *descs, int count, bool gated,
                                     ishi_projection **out) {
  if (!ctx || !out) return ISHI_E_INVALID;
  *out = nullptr;
  if (!descs) return fail(ctx, ISHI_E_INVALID, "null descriptor");
  if (count < 1 || count > kFragMaxSegments)
    return fail(ctx, ISHI_E_SHAPE, "%d weights in one projection, 1...%d are possible", count, kFragMaxSegments);
  int64_t wb = 0, n_total = 0;
  for (int i = 0; i < count; ++i) {
    int64_t part = 0;
    ishi_status s = check_desc(ctx, descs[i], &part);
    if (s != ISHI_OK) return s;
    const ishi_weight_desc &a = descs[0], &b = descs[i];
    if (a.kind != b.kind || a.ggml_type != b.ggml_type || a.bits != b.bits || a.group_size != b.group_size ||
        a.scale_dtype != b.scale_dtype || a.hadamard_block != b.hadamard_block || a.k != b.k || a.signs_dev != b.signs_dev)
      return fail(ctx, ISHI_E_SHAPE, "weight %d differs from weight 0 in format, input width or rotation", i);
    wb += part;
    n_total += b.n;
  }
  if (gated && (count != 2 || descs[0].n != descs[1].n || (descs[0].n & 7)))
    return fail(ctx, ISHI_E_SHAPE, "a gated pair needs two weights of the same height, a multiple of 8");
  std::lock_guard<std::mutex> g(ctx->lock);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  ishi_projection *p = new (std::nothrow) ishi_projection();
  if (!p) return fail(ctx, ISHI_E_NOMEM, "out of host memory");
  p->ctx = ctx;
  p->d = descs[0];
  p->d.n = n_total;  // the projection's weight rows: the weights stacked in the order given
  p->gated = gated;  // (or interleaved by eights, see FragSrc::pair_rows)
  p->fmt = format_of(descs[0]);
  p->weight_bytes = wb;
  ishi_status s = ISHI_OK;
  // Re-tile the weight once, for the kernel this format runs on; the caller's buffers are not read
  // again afterwards.
  std::vector<FragPlan> candidates;
  if (make_frag_plan(ctx, p->d, &p->frag, &candidates)) {
    s = ensure_workspace(ctx, &p->ws, 0, 0, p->frag.tiles_bytes, 0);
    if (s == ISHI_OK) s = tile_weight_frag(ctx, p->frag, descs, count, n_total, p->ws.tiles, 0, gated);
    if (s == ISHI_OK && !getenv("ISHI_NO_AUTOTUNE") && !getenv("ISHI_FRAG_PLAN")) tune_frag_plan(ctx, p, &candidates);
  } else if (count > 1) {
    delete p;
    return fail(ctx, ISHI_E_UNSUPPORTED, "only the warp-level kernel's formats can be stacked into one projection");
  } else if (make_row_plan(ctx, p->d, &p->plan)) {
    s = ensure_workspace(ctx, &p->ws, p->plan.scratch_floats, p->plan.counters, p->plan.tiles_bytes, 0);
    if (s == ISHI_OK) s = tile_weight(ctx, p->plan, p->d.n, p->ws.tiles, 0);
  } else if (p->d.kind == ISHI_KIND_GGML && !row_ops(p->fmt)) {
    // a block format without a streaming kernel: keep a plain copy of the blocks
    p->generic = true;
    s = ensure_workspace(ctx, &p->ws, 0, 0, (size_t)wb, 0);
    if (s == ISHI_OK && cudaMemcpyAsync(p->ws.tiles, descs[0].weight_dev, (size_t)wb, cudaMemcpyDeviceToDevice, 0) != cudaSuccess)
      s = fail(ctx, ISHI_E_CUDA, "copying the blocks failed");
  } else {
    delete p;
    return fail(ctx, ISHI_E_SHAPE, "no launch plan fits shared memory for k %lld", (long long)descs[0].k);
  }
  if (s == ISHI_OK) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) s = fail(ctx, ISHI_E_CUDA, "tiling the weight: %s", cudaGetErrorString(e));
  }
  if (s == ISHI_OK && p->d.hadamard_block != 0) {
    cudaError_t e = cudaMalloc(&p->xr, (size_t)16 * p->d.k * sizeof(__half));
    if (e != cudaSuccess) s = fail(ctx, ISHI_E_CUDA, "cudaMalloc(rotated x): %s", cudaGetErrorString(e));
  }
  // after create the library reads only its own tiled copy
  p->d.weight_dev = p->d.scales_dev = p->d.biases_dev = nullptr;
  if (s != ISHI_OK) {
    free_workspace(&p->ws);
    if (p->xr) cudaFree(p->xr);
    delete p;
    return s;
  }
  *out = p;
  return ISHI_OK;
}

ishi_status ishi_projection_create_fused(ishi_ctx *ctx, const ishi_weight_desc *descs, int count,
                                         ishi_projection **out) {
  return create_projection(ctx, descs, count, false, out);
}

ishi_status ishi_projection_create_gated(ishi_ctx *ctx, const ishi_weight_desc *gate, const ishi_weight_desc *up,
                                         ishi_projection **out) {
  if (!ctx || !out) return ISHI_E_INVALID;
  *out = nullptr;
  if (!gate || !up) return fail(ctx, ISHI_E_INVALID, "null descriptor");
  const ishi_weight_desc pair[2] = {*gate, *up};
  return create_projection(ctx, pair, 2, true, out);
}

ishi_status ishi_projection_create(ishi_ctx *ctx, const ishi_weight_desc *desc, ishi_projection **out) {
  return create_projection(ctx, desc, 1, false, out);
}

void ishi_projection_destroy(ishi_projection *p) {
  if (!p) return;
  cudaSetDevice(p->ctx->device);
  free_workspace(&p->ws);
  if (p->xr) cudaFree(p->xr);
  if (p->host_x) cudaFree(p->host_x);
  if (p->host_y) cudaFree(p->host_y);
  if (p->logits) cudaFree(p->logits);
  delete p;
}

int64_t ishi_projection_input_dim(const ishi_projection *p) { return p ? p->d.k : 0; }
int64_t ishi_projection_output_dim(const ishi_projection *p) { return p ? out_rows(p) : 0; }
int64_t ishi_projection_weight_bytes(const ishi_projection *p) { return p ? p->weight_bytes : 0; }
int ishi_projection_crossover_rows(const ishi_projection *p) {
  if (!p) return 0;
  return p->ctx->crossover_rows > 0 ? p->ctx->crossover_rows : 1;
}

ishi_status ishi_projection_plan(const ishi_projection *p, int plan[4]) {
  if (!p || !plan) return ISHI_E_INVALID;
  plan[0] = plan[1] = plan[2] = plan[3] = 0;
  if (p->frag.ok) plan[0] = p->frag.S, plan[1] = p->frag.Wu, plan[2] = p->frag.PP, plan[3] = p->frag.ring;
  return ISHI_OK;
}

ishi_status ishi_projection_set_plan(ishi_projection *p, const int plan[4]) {
  if (!p || !plan) return ISHI_E_INVALID;
  ishi_ctx *ctx = p->ctx;
  if (!p->frag.ok) return fail(ctx, ISHI_E_UNSUPPORTED, "this projection's kernel has one launch plan only");
  std::lock_guard<std::mutex> g(ctx->lock);
  ishi_weight_desc d = p->d;
  d.weight_dev = p->ws.tiles;  // the planner looks at sizes only
  std::vector<FragPlan> all;
  FragPlan best;
  if (!make_frag_plan(ctx, d, &best, &all)) return fail(ctx, ISHI_E_SHAPE, "no launch plan fits");
  for (const FragPlan &c : all)
    if (c.S == plan[0] && c.Wu == plan[1] && c.PP == plan[2] && c.ring == plan[3]) {
      p->frag = c;
      return ISHI_OK;
    }
  return fail(ctx, ISHI_E_INVALID, "plan %d,%d,%d,%d is not among this projection's launch plans", plan[0], plan[1], plan[2],
              plan[3]);
}

ishi_status ishi_projection_rotate(ishi_projection *p, const void *x, int rows, void *xr, void *stream) {
  if (!p) return ISHI_E_INVALID;
  ishi_ctx *ctx = p->ctx;
  if (!x || !xr) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (rows < 1) return fail(ctx, ISHI_E_SHAPE, "rows must be positive");
  if (p->d.hadamard_block == 0) {
    if (x != xr)
      ISHI_CUDA(ctx, cudaMemcpyAsync(xr, x, (size_t)rows * p->d.k * sizeof(__half), cudaMemcpyDeviceToDevice,
                                     static_cast<cudaStream_t>(stream)));
    return ISHI_OK;
  }
  return ishi_hadamard_rotate(ctx, x, rows, p->d.k, p->d.hadamard_block, p->d.signs_dev, xr, stream);
}

ishi_status ishi_projection_apply_rotated(ishi_projection *p, const void *xr, int rows, void *y, int64_t ldy,
                                          int flags, void *stream) {
  if (!p) return ISHI_E_INVALID;
  return projection_matmul(p, xr, rows, y, ldy, flags, false, static_cast<cudaStream_t>(stream));
}

ishi_status ishi_projection_apply(ishi_projection *p, const void *x, int rows, void *y, int64_t ldy, int flags,
                                  void *stream) {
  if (!p) return ISHI_E_INVALID;
  if (p->d.hadamard_block == 0)
    return projection_matmul(p, x, rows, y, ldy, flags, false, static_cast<cudaStream_t>(stream));
  if (rows < 1 || rows > 16) return fail(p->ctx, ISHI_E_SHAPE, "rows %d outside 1...16", rows);
  if (rotates_in_kernel(p) && getenv("ISHI_NO_FUSED_ROTATION") == nullptr)
    return projection_matmul(p, x, rows, y, ldy, flags, true, static_cast<cudaStream_t>(stream));
  ishi_status s = ishi_projection_rotate(p, x, rows, p->xr, stream);
  if (s != ISHI_OK) return s;
  return projection_matmul(p, p->xr, rows, y, ldy, flags, false, static_cast<cudaStream_t>(stream));
}

ishi_status ishi_projection_apply_argmax(ishi_projection *p, const void *x, int rows, int32_t *argmax_dev, void *stream) {
  if (!p) return ISHI_E_INVALID;
  ishi_ctx *ctx = p->ctx;
  if (!x || !argmax_dev) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (rows < 1 || rows > 16) return fail(ctx, ISHI_E_SHAPE, "rows %d outside 1...16", rows);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  if (!p->logits) {
    // the first call allocates the projection's logits buffer (make it outside stream capture)
    std::lock_guard<std::mutex> g(ctx->lock);
    if (!p->logits) {
      // [16][n] logits, then the arg-max kernel's scratch (its counters start at zero)
      __half *l = nullptr;
      const size_t logits_bytes = ((size_t)16 * out_rows(p) * sizeof(__half) + 255) & ~(size_t)255;
      if (cudaMalloc(&l, logits_bytes + argmax_scratch_bytes()) != cudaSuccess) return fail(ctx, ISHI_E_NOMEM, "logits buffer");
      if (cudaMemset(reinterpret_cast<uint8_t *>(l) + logits_bytes, 0, argmax_scratch_bytes()) != cudaSuccess) {
        cudaFree(l);
        return fail(ctx, ISHI_E_CUDA, "clearing the arg-max scratch failed");
      }
      p->logits = l;
    }
  }
  ishi_status s = ishi_projection_apply(p, x, rows, p->logits, out_rows(p), 0, stream);
  if (s != ISHI_OK) return s;
  const size_t logits_bytes = ((size_t)16 * out_rows(p) * sizeof(__half) + 255) & ~(size_t)255;
  ISHI_CUDA(ctx, launch_argmax_rows(p->logits, rows, out_rows(p), out_rows(p), argmax_dev,
                                    reinterpret_cast<uint8_t *>(p->logits) + logits_bytes, static_cast<cudaStream_t>(stream)));
  return ISHI_OK;
}

static ishi_status ensure_host_staging(ishi_projection *p);

ishi_status ishi_projection_apply_host_async(ishi_projection *p, const void *x_host, int rows, void *y_host,
                                             void *stream) {
  if (!p) return ISHI_E_INVALID;
  ishi_ctx *ctx = p->ctx;
  if (!x_host || !y_host) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (rows < 1 || rows > 16) return fail(ctx, ISHI_E_SHAPE, "rows %d outside 1...16", rows);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  {
    // the first call allocates this projection's device staging (make it outside stream capture)
    ishi_status s0 = ensure_host_staging(p);
    if (s0 != ISHI_OK) return s0;
  }
  const size_t xb = (size_t)rows * p->d.k * sizeof(__half), yb = (size_t)rows * out_rows(p) * sizeof(__half);
  ISHI_CUDA(ctx, cudaMemcpyAsync(p->host_x, x_host, xb, cudaMemcpyHostToDevice, st));
  ishi_status s = ishi_projection_apply(p, p->host_x, rows, p->host_y, out_rows(p), 0, stream);
  if (s != ISHI_OK) return s;
  ISHI_CUDA(ctx, cudaMemcpyAsync(y_host, p->host_y, yb, cudaMemcpyDeviceToHost, st));
  return ISHI_OK;
}

// device staging of the host-buffer entry points: [16][k] and [16][n], allocated by the first call
static ishi_status ensure_host_staging(ishi_projection *p) {
  ishi_ctx *ctx = p->ctx;
  if (p->host_x) return ISHI_OK;
  std::lock_guard<std::mutex> g(ctx->lock);
  if (p->host_x) return ISHI_OK;
  __half *hx = nullptr, *hy = nullptr;
  ISHI_CUDA(ctx, cudaMalloc(&hx, (size_t)16 * p->d.k * sizeof(__half)));
  cudaError_t e = cudaMalloc(&hy, (size_t)16 * out_rows(p) * sizeof(__half));
  if (e != cudaSuccess) {
    cudaFree(hx);
    return fail(ctx, ISHI_E_NOMEM, "device staging: %s", cudaGetErrorString(e));
  }
  p->host_y = hy;
  p->host_x = hx;
  return ISHI_OK;
}

ishi_status ishi_projection_apply_host_batch(ishi_projection *const *ps, const void *const *x_hosts, int rows,
                                             void *const *y_hosts, int count, void *stream) {
  if (!ps || count < 1 || !ps[0]) return ISHI_E_INVALID;
  ishi_ctx *ctx = ps[0]->ctx;
  if (!x_hosts || !y_hosts) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (rows < 1 || rows > 16) return fail(ctx, ISHI_E_SHAPE, "rows %d outside 1...16", rows);
  for (int i = 0; i < count; ++i) {
    if (!ps[i] || !x_hosts[i] || !y_hosts[i]) return fail(ctx, ISHI_E_INVALID, "null pointer in entry %d", i);
    if (ps[i]->ctx != ctx) return fail(ctx, ISHI_E_INVALID, "projection %d belongs to another context", i);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  {
    std::lock_guard<std::mutex> g(ctx->lock);
    if (!ctx->copy_in) {
      ISHI_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking));
      ISHI_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking));
      ISHI_CUDA(ctx, cudaEventCreateWithFlags(&ctx->ev_begin, cudaEventDisableTiming));
      ISHI_CUDA(ctx, cudaEventCreateWithFlags(&ctx->ev_end, cudaEventDisableTiming));
    }
    while ((int)ctx->ev_in.size() < count) {
      cudaEvent_t a = nullptr, b = nullptr;
      ISHI_CUDA(ctx, cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
      ctx->ev_in.push_back(a);
      ISHI_CUDA(ctx, cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
      ctx->ev_done.push_back(b);
    }
  }
  for (int i = 0; i < count; ++i) {
    ishi_status s = ensure_host_staging(ps[i]);
    if (s != ISHI_OK) return s;
  }
  // Three lanes: x copies run ahead on one stream, the products follow on the caller's stream as
  // their inputs land, the y copies trail on a third; the caller's stream ends behind all of them.
  // The lanes hand over in chunks of kChunk entries, not entry by entry: an event between two
  // product kernels would serialise them, inside a chunk they follow each other with programmatic
  // dependent launch as in a plain sequence of applies.
  constexpr int kChunk = 16;
  ISHI_CUDA(ctx, cudaEventRecord(ctx->ev_begin, st));
  ISHI_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_in, ctx->ev_begin, 0));
  ISHI_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, ctx->ev_begin, 0));
  for (int c0 = 0; c0 < count; c0 += kChunk) {
    const int c1 = std::min(count, c0 + kChunk);
    for (int i = c0; i < c1; ++i) {
      const size_t xb = (size_t)rows * ps[i]->d.k * sizeof(__half);
      ISHI_CUDA(ctx, cudaMemcpyAsync(ps[i]->host_x, x_hosts[i], xb, cudaMemcpyHostToDevice, ctx->copy_in));
    }
    ISHI_CUDA(ctx, cudaEventRecord(ctx->ev_in[c0], ctx->copy_in));
    ISHI_CUDA(ctx, cudaStreamWaitEvent(st, ctx->ev_in[c0], 0));
    for (int i = c0; i < c1; ++i) {
      ishi_status s = ishi_projection_apply(ps[i], ps[i]->host_x, rows, ps[i]->host_y, out_rows(ps[i]), 0, stream);
      if (s != ISHI_OK) return s;
    }
    ISHI_CUDA(ctx, cudaEventRecord(ctx->ev_done[c0], st));
    ISHI_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, ctx->ev_done[c0], 0));
    for (int i = c0; i < c1; ++i) {
      const size_t yb = (size_t)rows * out_rows(ps[i]) * sizeof(__half);
      ISHI_CUDA(ctx, cudaMemcpyAsync(y_hosts[i], ps[i]->host_y, yb, cudaMemcpyDeviceToHost, ctx->copy_out));
    }
  }
  ISHI_CUDA(ctx, cudaEventRecord(ctx->ev_end, ctx->copy_out));
  ISHI_CUDA(ctx, cudaStreamWaitEvent(st, ctx->ev_end, 0));
  return ISHI_OK;
}

ishi_status ishi_projection_apply_host(ishi_projection *p, const void *x_host, int rows, void *y_host, void *stream) {
  if (!p) return ISHI_E_INVALID;
  ishi_ctx *ctx = p->ctx;
  if (!x_host || !y_host) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (rows < 1 || rows > 16) return fail(ctx, ISHI_E_SHAPE, "rows %d outside 1...16", rows);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t xb = (size_t)rows * p->d.k * sizeof(__half), yb = (size_t)rows * out_rows(p) * sizeof(__half);
  {
    std::lock_guard<std::mutex> g(ctx->lock);
    ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
    if (xb > ctx->pin_x_bytes) {
      if (ctx->pin_x) cudaFreeHost(ctx->pin_x);
      if (ctx->dev_x) cudaFree(ctx->dev_x);
      ctx->pin_x = ctx->dev_x = nullptr;
      ctx->pin_x_bytes = 0;
      const size_t cap = (size_t)16 * p->d.k * sizeof(__half);
      ISHI_CUDA(ctx, cudaHostAlloc(&ctx->pin_x, cap, cudaHostAllocDefault));
      ISHI_CUDA(ctx, cudaMalloc(&ctx->dev_x, cap));
      ctx->pin_x_bytes = cap;
    }
    if (yb > ctx->pin_y_bytes) {
      if (ctx->pin_y) cudaFreeHost(ctx->pin_y);
      if (ctx->dev_y) cudaFree(ctx->dev_y);
      ctx->pin_y = ctx->dev_y = nullptr;
      ctx->pin_y_bytes = 0;
      const size_t cap = (size_t)16 * out_rows(p) * sizeof(__half);
      ISHI_CUDA(ctx, cudaHostAlloc(&ctx->pin_y, cap, cudaHostAllocDefault));
      ISHI_CUDA(ctx, cudaMalloc(&ctx->dev_y, cap));
      ctx->pin_y_bytes = cap;
    }
  }
  memcpy(ctx->pin_x, x_host, xb);
  ISHI_CUDA(ctx, cudaMemcpyAsync(ctx->dev_x, ctx->pin_x, xb, cudaMemcpyHostToDevice, st));
  ishi_status s = ishi_projection_apply(p, ctx->dev_x, rows, ctx->dev_y, out_rows(p), 0, stream);
  if (s != ISHI_OK) return s;
  ISHI_CUDA(ctx, cudaMemcpyAsync(ctx->pin_y, ctx->dev_y, yb, cudaMemcpyDeviceToHost, st));
  ISHI_CUDA(ctx, cudaStreamSynchronize(st));
  memcpy(y_host, ctx->pin_y, yb);
  return ishi_ctx_poll(ctx);
}

}  // extern "C"

// ---- output exchange between the GPUs of an N-sharded projection ---------------------------------

struct ishi_exchange {
  ishi_ctx *ctx = nullptr;
  int rank = 0, world = 1;
  uint8_t *buf = nullptr;
  size_t bytes = 0;
  unsigned *words = nullptr;  // [0, world): arrival words; [16]: CTAs done; [17]: number of the last launch
  uint8_t *peer_buf[kFragMaxPeers] = {nullptr};
  unsigned *peer_words[kFragMaxPeers] = {nullptr};
  bool connected = false;
};

struct ExchangeHandle {
  cudaIpcMemHandle_t buf, words;
};
static_assert(sizeof(ExchangeHandle) <= ISHI_EXCHANGE_HANDLE_BYTES, "two IPC handles fit the exported blob");

ishi_status ishi_exchange_create(ishi_ctx *ctx, int rank, int world, int64_t out_bytes, ishi_exchange **out) {
  if (!ctx || !out) return ISHI_E_INVALID;
  *out = nullptr;
  if (world < 1 || world > kFragMaxPeers || rank < 0 || rank >= world || out_bytes < 16)
    return fail(ctx, ISHI_E_INVALID, "exchange of rank %d of %d, %lld bytes", rank, world, (long long)out_bytes);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  ishi_exchange *ex = new (std::nothrow) ishi_exchange();
  if (!ex) return fail(ctx, ISHI_E_NOMEM, "host allocation failed");
  ex->ctx = ctx;
  ex->rank = rank;
  ex->world = world;
  ex->bytes = (size_t)out_bytes;
  cudaError_t e = cudaMalloc(&ex->buf, ex->bytes);
  if (e == cudaSuccess) e = cudaMalloc(&ex->words, 256);
  if (e == cudaSuccess) e = cudaMemset(ex->words, 0, 256);
  if (e == cudaSuccess) e = cudaMemset(ex->buf, 0, ex->bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    if (ex->buf) cudaFree(ex->buf);
    if (ex->words) cudaFree(ex->words);
    delete ex;
    return fail(ctx, ISHI_E_NOMEM, "exchange buffers: %s", cudaGetErrorString(e));
  }
  ex->peer_buf[rank] = ex->buf;
  ex->peer_words[rank] = ex->words;
  ex->connected = world == 1;
  *out = ex;
  return ISHI_OK;
}

ishi_status ishi_exchange_export(ishi_exchange *ex, void *handle_out) {
  if (!ex || !handle_out) return ISHI_E_INVALID;
  ishi_ctx *ctx = ex->ctx;
  ExchangeHandle h;
  memset(&h, 0, sizeof(h));
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  ISHI_CUDA(ctx, cudaIpcGetMemHandle(&h.buf, ex->buf));
  ISHI_CUDA(ctx, cudaIpcGetMemHandle(&h.words, ex->words));
  memset(handle_out, 0, ISHI_EXCHANGE_HANDLE_BYTES);
  memcpy(handle_out, &h, sizeof(h));
  return ISHI_OK;
}

ishi_status ishi_exchange_connect(ishi_exchange *ex, const void *handles) {
  if (!ex || !handles) return ISHI_E_INVALID;
  ishi_ctx *ctx = ex->ctx;
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  for (int q = 0; q < ex->world; ++q) {
    if (q == ex->rank || ex->peer_buf[q]) continue;
    ExchangeHandle h;
    memcpy(&h, static_cast<const uint8_t *>(handles) + (size_t)q * ISHI_EXCHANGE_HANDLE_BYTES, sizeof(h));
    void *b = nullptr, *w = nullptr;
    ISHI_CUDA(ctx, cudaIpcOpenMemHandle(&b, h.buf, cudaIpcMemLazyEnablePeerAccess));
    ISHI_CUDA(ctx, cudaIpcOpenMemHandle(&w, h.words, cudaIpcMemLazyEnablePeerAccess));
    ex->peer_buf[q] = static_cast<uint8_t *>(b);
    ex->peer_words[q] = static_cast<unsigned *>(w);
  }
  ex->connected = true;
  return ISHI_OK;
}

void *ishi_exchange_buffer(ishi_exchange *ex) { return ex ? ex->buf : nullptr; }

ishi_status ishi_exchange_apply(ishi_exchange *ex, ishi_projection *p, const void *x, int rows, int64_t out_offset_bytes,
                                int64_t row_offset, int wait_previous, void *stream) {
  if (!ex || !p) return ISHI_E_INVALID;
  ishi_ctx *ctx = ex->ctx;
  if (p->ctx != ctx) return fail(ctx, ISHI_E_INVALID, "projection and exchange belong to different contexts");
  if (!ex->connected) return fail(ctx, ISHI_E_INVALID, "exchange not connected");
  if (!x) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (!p->frag.ok) {
    // The other kernels do not store to peers themselves: the product goes into this rank's own
    // copy and a small kernel passes the rows on and publishes them.
    if (rows < 1 || rows > 8) return fail(ctx, ISHI_E_SHAPE, "rows %d outside 1...8 for this weight format", rows);
    if (p->d.hadamard_block != 0) return fail(ctx, ISHI_E_UNSUPPORTED, "a rotated pack of this format cannot be exchanged");
    if (out_offset_bytes < 0 || (out_offset_bytes & 15) || row_offset < 0 ||
        (size_t)out_offset_bytes + (size_t)(row_offset + p->d.n) * 16 > ex->bytes)
      return fail(ctx, ISHI_E_SHAPE, "rows %lld...%lld at offset %lld do not fit the exchange buffer", (long long)row_offset,
                  (long long)(row_offset + p->d.n), (long long)out_offset_bytes);
    ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (wait_previous) {
      peer_wait_kernel<<<1, 32, 0, st>>>(ex->words, ex->world, ex->words + 17, ctx->err_dev);
      ISHI_CUDA(ctx, cudaGetLastError());
    }
    __half *mine = reinterpret_cast<__half *>(ex->buf + out_offset_bytes);
    ishi_status s = projection_matmul(p, x, rows, mine + row_offset * 8, 8, ISHI_OUT_TRANSPOSED, false, st);
    if (s != ISHI_OK) return s;
    PublishArgs pa;
    memset(&pa, 0, sizeof(pa));
    for (int q = 0; q < ex->world; ++q) {
      pa.peer_y[q] = reinterpret_cast<__half *>(ex->peer_buf[q] + out_offset_bytes);
      pa.peer_flags[q] = ex->peer_words[q];
    }
    pa.done = ex->words + 16;
    pa.launch_no = ex->words + 17;
    pa.first = row_offset;
    pa.n = p->d.n;
    pa.world = ex->world;
    pa.rank = ex->rank;
    pa.M = rows;
    const int grid = (int)std::min<long long>((p->d.n + 255) / 256, ctx->sm_count);
    publish_rows_kernel<<<grid, 256, 0, st>>>(pa);
    ISHI_CUDA(ctx, cudaGetLastError());
    return ISHI_OK;
  }
  if (rows < 1 || rows > 16) return fail(ctx, ISHI_E_SHAPE, "rows %d outside 1...16", rows);
  const size_t row_bytes = rows > 8 ? 32 : 16;
  if (out_offset_bytes < 0 || (out_offset_bytes & 15) || row_offset < 0 ||
      (size_t)out_offset_bytes + (size_t)(row_offset + out_rows(p)) * row_bytes > ex->bytes)
    return fail(ctx, ISHI_E_SHAPE, "rows %lld...%lld at offset %lld do not fit the exchange buffer", (long long)row_offset,
                (long long)(row_offset + out_rows(p)), (long long)out_offset_bytes);
  const int b = p->d.hadamard_block;
  if (b != 0 && !rotates_in_kernel(p)) return fail(ctx, ISHI_E_UNSUPPORTED, "rotation block %d needs its own kernel", b);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  PeerOut po;
  memset(&po, 0, sizeof(po));
  po.world = ex->world;
  po.rank = ex->rank;
  for (int q = 0; q < ex->world; ++q) {
    po.y[q] = reinterpret_cast<__half *>(ex->peer_buf[q] + out_offset_bytes);
    po.flags[q] = ex->peer_words[q];
  }
  po.local_flags = ex->words;
  po.done = ex->words + 16;
  po.launch_no = ex->words + 17;
  po.wait_previous = wait_previous ? 1 : 0;
  po.row_offset = row_offset;
  return run_frag(ctx, p->frag, p->ws, p->d, x, rows, ex->buf + out_offset_bytes, rows > 8 ? 16 : 8, ISHI_OUT_TRANSPOSED, false,
                  getenv("ISHI_NO_EARLY_LAUNCH") == nullptr, b != 0, static_cast<cudaStream_t>(stream), &po, p->gated);
}

ishi_status ishi_exchange_wait(ishi_exchange *ex, void *stream) {
  if (!ex) return ISHI_E_INVALID;
  ishi_ctx *ctx = ex->ctx;
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  peer_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ex->words, ex->world, ex->words + 17, ctx->err_dev);
  ISHI_CUDA(ctx, cudaGetLastError());
  return ISHI_OK;
}

ishi_status ishi_exchange_debug_expect(ishi_exchange *ex, unsigned launches_ahead) {
  if (!ex) return ISHI_E_INVALID;
  ishi_ctx *ctx = ex->ctx;
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  unsigned seq = 0;
  ISHI_CUDA(ctx, cudaMemcpy(&seq, ex->words + 17, sizeof(seq), cudaMemcpyDeviceToHost));
  seq += launches_ahead;
  ISHI_CUDA(ctx, cudaMemcpy(ex->words + 17, &seq, sizeof(seq), cudaMemcpyHostToDevice));
  return ISHI_OK;
}

ishi_status ishi_exchange_disconnect(ishi_exchange *ex) {
  if (!ex) return ISHI_E_INVALID;
  cudaSetDevice(ex->ctx->device);
  // this rank's launches may still be storing into the peers' buffers
  if (cudaDeviceSynchronize() != cudaSuccess) return fail(ex->ctx, ISHI_E_CUDA, "synchronising before the disconnect failed");
  for (int q = 0; q < ex->world; ++q) {
    if (q == ex->rank) continue;
    if (ex->peer_buf[q]) cudaIpcCloseMemHandle(ex->peer_buf[q]);
    if (ex->peer_words[q]) cudaIpcCloseMemHandle(ex->peer_words[q]);
    ex->peer_buf[q] = nullptr;
    ex->peer_words[q] = nullptr;
  }
  ex->connected = false;
  return ISHI_OK;
}

void ishi_exchange_destroy(ishi_exchange *ex) {
  if (!ex) return;
  ishi_exchange_disconnect(ex);
  if (ex->buf) cudaFree(ex->buf);
  if (ex->words) cudaFree(ex->words);
  delete ex;
}

// ---- the entry point for callers that cannot allocate ---------------------------------------------
//
// Everything rowstream_kernel needs beyond the caller's x, blocks and y sits in this one array,
// which is part of the library image on every GPU that loads it:
//   [0, 16 KiB)        arrival counters, one per (panel, warp): at most 1024 panels
//   [16 KiB, 64 KiB)   the error word a bounded wait raises (first 4 bytes)
//   [64 KiB, 4 MiB)    fp32 partial sums of panels shared between CTAs
//   [4 MiB, 16 MiB)    the weight re-tiled for the kernel
// On the host the symbol below is only a stand-in: its device address comes from
// cudaGetSymbolAddress, once per device, and that address is what the kernels are given.
namespace {
constexpr size_t kStaticBytes = 16u << 20;
constexpr size_t kStaticCounters = 0, kStaticCountersBytes = 16u << 10;
constexpr size_t kStaticErr = 16u << 10;
constexpr size_t kStaticPartials = 64u << 10, kStaticPartialsBytes = (4u << 20) - (64u << 10);
constexpr size_t kStaticTiles = 4u << 20, kStaticTilesBytes = 12u << 20;
}  // namespace

static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

extern "C" ishi_status ishi_q4k_matmul_few_static(const void *x, int rows, const void *blocks, int64_t blocks_bytes,
                                                  int64_t n, int64_t k, void *y, void *stream) {
  static unsigned char *base[64] = {nullptr};  // device address of the array, per device
  static std::mutex setup_lock;

  ishi_ctx tmp;  // a stack record for the helpers; nothing in it owns memory
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return ISHI_E_CUDA;
  tmp.device = dev;
  int major = 0;
  if (cudaDeviceGetAttribute(&tmp.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&tmp.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
    return ISHI_E_CUDA;
  if (major != 10) return ISHI_E_UNSUPPORTED;  // the kernels are built for sm_100a only

  ishi_status s = check_io(&tmp, x, rows, y, 16);
  if (s != ISHI_OK) return s;
  ishi_weight_desc d;
  memset(&d, 0, sizeof(d));
  d.kind = ISHI_KIND_GGML;
  d.ggml_type = ISHI_GGML_Q4_K;
  d.n = n;
  d.k = k;
  d.weight_dev = blocks;
  d.weight_bytes = blocks_bytes;
  int64_t wb = 0;
  s = check_desc(&tmp, d, &wb);
  if (s != ISHI_OK) return s;
  RowPlan pl;
  if (!make_row_plan(&tmp, d, &pl)) return ISHI_E_SHAPE;
  if (pl.counters * sizeof(unsigned int) > kStaticCountersBytes || pl.scratch_floats * sizeof(float) > kStaticPartialsBytes ||
      pl.tiles_bytes > kStaticTilesBytes)
    return ISHI_E_TOO_LARGE;

  unsigned char *b = nullptr;
  {
    std::lock_guard<std::mutex> g(setup_lock);
    if (base[dev] == nullptr) {
      void *p = nullptr;
      if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return ISHI_E_CUDA;
      base[dev] = static_cast<unsigned char *>(p);
    }
    b = base[dev];
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the counters must start at zero and the error word clear, whatever the last call left behind
  if (cudaMemsetAsync(b + kStaticCounters, 0, kStaticCountersBytes + 64, st) != cudaSuccess) return ISHI_E_CUDA;

  Workspace ws;
  ws.counters = reinterpret_cast<unsigned int *>(b + kStaticCounters);
  ws.scratch = reinterpret_cast<float *>(b + kStaticPartials);
  ws.tiles = b + kStaticTiles;
  tmp.err_dev = reinterpret_cast<int *>(b + kStaticErr);
  s = tile_weight(&tmp, pl, n, ws.tiles, st);
  if (s == ISHI_OK) s = run_rows(&tmp, pl, ws, ISHI_GGML_Q4_K, d, x, rows, y, n, 0, st);
  ws = Workspace();  // nothing here was allocated, nothing to free
  if (s != ISHI_OK) return s;
  if (cudaStreamSynchronize(st) != cudaSuccess) return ISHI_E_CUDA;
  int raised = 0;
  if (cudaMemcpy(&raised, b + kStaticErr, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return ISHI_E_CUDA;
  return raised ? ISHI_E_TIMEOUT : ISHI_OK;
}

ishi_status ishi_rms_norm(ishi_ctx *ctx, const void *x, int x_dtype, int64_t rows, int64_t width, const void *weight,
                          int weight_dtype, float eps, void *y, void *stream) {
  if (!ctx) return ISHI_E_INVALID;
  if (!x || !weight || !y) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if ((x_dtype != ISHI_DT_F16 && x_dtype != ISHI_DT_F32) || weight_dtype < ISHI_DT_F16 || weight_dtype > ISHI_DT_F32)
    return fail(ctx, ISHI_E_INVALID, "bad dtype");
  if (rows < 0 || rows > 65535 || width <= 0 || width > rms_norm_max_width())
    return fail(ctx, ISHI_E_SHAPE, "rows %lld or width %lld outside this kernel's range (width <= %lld)", (long long)rows,
                (long long)width, rms_norm_max_width());
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  ISHI_CUDA(ctx, launch_rms_norm(x, x_dtype, weight, weight_dtype, rows, width, eps, static_cast<__half *>(y),
                                 static_cast<cudaStream_t>(stream)));
  return ISHI_OK;
}

// ---- EXL3 -----------------------------------------------------------------------------------------

namespace {
// EXL3Tensor.init's guards (Sources/IshizukiKit/Core/EXL3.swift:28-49)
ishi_status check_exl3(ishi_ctx *ctx, const ishi_exl3_desc *t, bool need_scales) {
  if (!t || !t->trellis_dev) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (reinterpret_cast<uintptr_t>(t->trellis_dev) & 3u) return fail(ctx, ISHI_E_INVALID, "trellis not 4-byte aligned");
  if (!exl3_rate_supported(t->words_per_tile, t->codebook))
    return fail(ctx, ISHI_E_UNSUPPORTED, "an EXL3 tile of %d words with codebook %d is not a rate", t->words_per_tile, t->codebook);
  if (t->k <= 0 || t->n <= 0 || t->k % 128 != 0 || t->n % 128 != 0 || t->k > (1ll << 24) || t->n > (1ll << 24))
    return fail(ctx, ISHI_E_SHAPE, "EXL3 %lldx%lld is not a whole number of 128 blocks", (long long)t->k, (long long)t->n);
  if (need_scales && (!t->input_scales_dev || !t->output_scales_dev)) return fail(ctx, ISHI_E_INVALID, "null scale vector");
  return ISHI_OK;
}
}  // namespace

ishi_status ishi_exl3_dequantize(ishi_ctx *ctx, const ishi_exl3_desc *t, int out_dtype, void *w_out, void *stream) {
  if (!ctx) return ISHI_E_INVALID;
  ishi_status s = check_exl3(ctx, t, false);
  if (s != ISHI_OK) return s;
  if (!w_out) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (out_dtype != ISHI_DT_F16 && out_dtype != ISHI_DT_F32) return fail(ctx, ISHI_E_INVALID, "bad output dtype %d", out_dtype);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  ISHI_CUDA(ctx, launch_exl3_dequantize(t->trellis_dev, (int)(t->k / 16), (int)(t->n / 16), t->words_per_tile, t->codebook, w_out,
                                        out_dtype, ctx->sm_count, static_cast<cudaStream_t>(stream)));
  return ISHI_OK;
}

ishi_status ishi_exl3_rotate(ishi_ctx *ctx, const void *x, int x_dtype, int64_t rows, int64_t width, const void *scales_dev,
                             int before, void *y, int y_dtype, void *stream) {
  if (!ctx) return ISHI_E_INVALID;
  if (!x || !y || !scales_dev) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if ((x_dtype != ISHI_DT_F16 && x_dtype != ISHI_DT_F32) || (y_dtype != ISHI_DT_F16 && y_dtype != ISHI_DT_F32))
    return fail(ctx, ISHI_E_INVALID, "bad dtype");
  if (rows < 0 || width <= 0 || width % 128 != 0) return fail(ctx, ISHI_E_SHAPE, "width %lld is not a whole number of 128 blocks", (long long)width);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  ISHI_CUDA(ctx, launch_exl3_rotate(x, x_dtype, rows, width, static_cast<const __half *>(scales_dev), before ? 1 : 0, y, y_dtype,
                                    ctx->sm_count, static_cast<cudaStream_t>(stream)));
  return ISHI_OK;
}

ishi_status ishi_exl3_matvec(ishi_ctx *ctx, const ishi_exl3_desc *t, const void *x, int rows, float *y, void *stream) {
  if (!ctx) return ISHI_E_INVALID;
  ishi_status s = check_exl3(ctx, t, false);
  if (s != ISHI_OK) return s;
  if (!x || !y) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (reinterpret_cast<uintptr_t>(x) & 3u) return fail(ctx, ISHI_E_INVALID, "x must be 4-byte aligned");
  if (rows < 1 || rows > 8) return fail(ctx, ISHI_E_SHAPE, "rows %d outside 1...8", rows);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  ISHI_CUDA(ctx, launch_exl3_matvec(t->trellis_dev, (int)(t->k / 16), (int)(t->n / 16), t->words_per_tile, t->codebook,
                                    static_cast<const __half *>(x), rows, y, ctx->sm_count, static_cast<cudaStream_t>(stream)));
  return ISHI_OK;
}

ishi_status ishi_exl3_apply(ishi_ctx *ctx, const ishi_exl3_desc *t, const void *x, int rows, void *y, void *stream) {
  if (!ctx) return ISHI_E_INVALID;
  ishi_status s = check_exl3(ctx, t, true);
  if (s != ISHI_OK) return s;
  if (!x || !y) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (rows < 1 || rows > 16) return fail(ctx, ISHI_E_SHAPE, "rows %d outside 1...16", rows);
  std::lock_guard<std::mutex> g(ctx->lock);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t xb = (size_t)16 * t->k * sizeof(__half), yb = (size_t)16 * t->n * sizeof(float);
  if (ctx->exl3_x_cap < xb) {
    ISHI_CUDA(ctx, cudaStreamSynchronize(st));  // earlier calls may still read the smaller buffer
    if (ctx->exl3_x) cudaFree(ctx->exl3_x);
    ctx->exl3_x = nullptr, ctx->exl3_x_cap = 0;
    ISHI_CUDA(ctx, cudaMalloc(&ctx->exl3_x, xb));
    ctx->exl3_x_cap = xb;
  }
  if (ctx->exl3_y_cap < yb) {
    ISHI_CUDA(ctx, cudaStreamSynchronize(st));
    if (ctx->exl3_y) cudaFree(ctx->exl3_y);
    ctx->exl3_y = nullptr, ctx->exl3_y_cap = 0;
    ISHI_CUDA(ctx, cudaMalloc(&ctx->exl3_y, yb));
    ctx->exl3_y_cap = yb;
  }
  ISHI_CUDA(ctx, launch_exl3_rotate(x, ISHI_DT_F16, rows, t->k, static_cast<const __half *>(t->input_scales_dev), 1, ctx->exl3_x,
                                    ISHI_DT_F16, ctx->sm_count, st));
  for (int r0 = 0; r0 < rows; r0 += 8)
    ISHI_CUDA(ctx, launch_exl3_matvec(t->trellis_dev, (int)(t->k / 16), (int)(t->n / 16), t->words_per_tile, t->codebook,
                                      ctx->exl3_x + (size_t)r0 * t->k, std::min(8, rows - r0), ctx->exl3_y + (size_t)r0 * t->n, ctx->sm_count, st));
  ISHI_CUDA(ctx, launch_exl3_rotate(ctx->exl3_y, ISHI_DT_F32, rows, t->n, static_cast<const __half *>(t->output_scales_dev), 0, y,
                                    ISHI_DT_F16, ctx->sm_count, st));
  return ISHI_OK;
}
