// C ABI of the verify-matmul library: argument validation, per-shape launch plans, the
// row-count crossover and the kernel launches. No torch, no NCCL, no CPU fallback: a shape
// without a kernel is an error status.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>

#include "../../include/ishizuki_cuda.h"
#include "dequant.cuh"
#include "fmt_q4k.cuh"
#include "ishi_stream.cuh"
#include "rfmt_q4k.cuh"

using namespace ishi;

namespace {

constexpr int kSmemBudget = 227 * 1024 - 512;  // dynamic part; the kernels also hold a few static bytes

struct Workspace {
  float *scratch = nullptr;
  unsigned int *counters = nullptr;
  size_t scratch_floats = 0;
  size_t n_counters = 0;
};

}  // namespace

struct ishi_ctx {
  int device = 0;
  int sm_count = 0;
  int smem_optin = 0;
  int route = ISHI_ROUTE_AUTO;
  int crossover_rows = 0;
  int *err_host = nullptr;  // mapped pinned word the kernels raise on a timed-out wait
  int *err_dev = nullptr;
  Workspace ws;             // for the kernel-level entry points
  void *pin_x = nullptr, *pin_y = nullptr;  // pinned staging for apply_host
  void *dev_x = nullptr, *dev_y = nullptr;
  size_t pin_x_bytes = 0, pin_y_bytes = 0;
  std::mutex lock;
  char last_error[256] = {0};
};

namespace {

struct Plan;

}  // namespace

namespace {

struct Plan {
  int fmt = 0;  // ggml type, or 100 + bits for affine
  int units = 0, S = 1, P = 0, Gc = 1, SL = 2, W = 1, UW = 1, MT = 1, nstages = 2, row_stride = 0;
  int seg_off[kMaxSrc] = {0, 0, 0};
  size_t smem = 0;
  size_t scratch_floats = 0;
};

ishi_status fail(ishi_ctx *ctx, ishi_status s, const char *fmt, ...) {
  if (ctx) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(ctx->last_error, sizeof(ctx->last_error), fmt, ap);
    va_end(ap);
  }
  return s;
}

#define ISHI_CUDA(ctx, call)                                                             \
  do {                                                                                   \
    cudaError_t e_ = (call);                                                             \
    if (e_ != cudaSuccess)                                                               \
      return fail(ctx, ISHI_E_CUDA, "%s: %s", #call, cudaGetErrorString(e_));            \
  } while (0)

int type_size(int t) {
  switch (t) {
    case ISHI_GGML_Q4_K: return 144;
    case ISHI_GGML_Q6_K: return 210;
    case ISHI_GGML_IQ2_XS: return 74;
    default: return 0;
  }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Fixes the grid, the K split and the shared-memory ring for one (format, N, K, rows) shape.
// unit_bytes[i] are the per-row bytes of each byte stream for one 256-wide unit.
bool make_plan(const ishi_ctx *ctx, int fmt, long long N, long long K, int rows, int nsrc,
               const int *unit_bytes, int row_skew, Plan *pl) {
  pl->fmt = fmt;
  pl->MT = rows > 8 ? 2 : 1;
  pl->UW = rows > 8 ? 1 : 2;
  pl->units = (int)(K / 256);
  pl->P = (int)((N + kPanelRows - 1) / kPanelRows);
  const int cap = kMaxConsumerWarps * pl->UW;
  const int smin = (pl->units + cap - 1) / cap;
  // Among the few smallest workable splits take the one that occupies the most SMs.
  int best_s = smin, best_g = 0;
  for (int s = smin; s <= std::min(pl->units, smin + 3); ++s) {
    if (s > ctx->sm_count) break;
    const int g = (ctx->sm_count / s) * s;
    if (g > best_g) {
      best_g = g;
      best_s = s;
    }
  }
  pl->S = best_s;
  pl->Gc = std::max(1, ctx->sm_count / pl->S);
  const int umax = (pl->units + pl->S - 1) / pl->S;
  pl->W = (umax + pl->UW - 1) / pl->UW;
  const int dense_slots = (pl->Gc + pl->P - 1) / pl->P + 1;
  pl->SL = (long long)pl->P * (pl->units / pl->S) >= pl->Gc ? dense_slots : std::max(umax, dense_slots);
  int need = 0;
  for (int i = 0; i < nsrc; ++i) {
    pl->seg_off[i] = need;
    need += (umax * unit_bytes[i] + 30 + 15) & ~15;
  }
  int stride = (need + 127) / 128 * 128 + row_skew;
  if (stride - 128 >= need) stride -= 128;
  pl->row_stride = stride;
  const size_t stage = (size_t)kPanelRows * stride;
  int nst = 8;
  for (; nst >= 2; --nst) {
    const size_t bars = ((size_t)(2 * nst + nst + 1) * 8 + 127) & ~(size_t)127;
    const size_t red = (size_t)(nst + 1) * pl->W * pl->MT * 512;
    pl->smem = bars + red + nst * stage;
    if (pl->smem <= (size_t)std::min(kSmemBudget, ctx->smem_optin)) break;
  }
  if (nst < 2) return false;
  pl->nstages = nst;
  pl->scratch_floats = (size_t)pl->P * pl->S * pl->SL * 2 /* room for 16 rows */ * 128;
  return true;
}

// Launch plan of the tcgen05 kernel (rows 1...8): two CTAs per SM, 128-row panels, kc units per
// stage, the weight read from its tiled copy.
struct RowPlan {
  bool ok = false;
  int units = 0, P = 0, SL = 2, kc = 2, nstages = 2, x_off = 0, bmin_off = 0, stage_bytes = 0;
  int grid = 0, nsrc = 0;
  int tile_bytes = 0, sec_off[kMaxSrc] = {0, 0, 0}, unit_bytes[kMaxSrc] = {0, 0, 0};
  size_t smem = 0, scratch_floats = 0, counters = 0, tiles_bytes = 0;
};

bool make_row_plan(const ishi_ctx *ctx, long long N, long long K, int nsrc, const int *unit_bytes, RowPlan *pl) {
  pl->units = (int)(K / 256);
  pl->P = (int)((N + kRowPanel - 1) / kRowPanel);
  pl->grid = 2 * ctx->sm_count;
  pl->nsrc = nsrc;
  int tile = 0;
  for (int i = 0; i < nsrc; ++i) {
    pl->sec_off[i] = tile;
    pl->unit_bytes[i] = unit_bytes[i];
    tile += kRowPanel * unit_bytes[i];  // a multiple of 128 bytes
  }
  pl->tile_bytes = tile;
  pl->tiles_bytes = (size_t)pl->P * pl->units * tile;
  const size_t half_sm = (size_t)(std::min(kSmemBudget, ctx->smem_optin) - 2048) / 2;
  // two units a stage when they fit twice, else one
  for (pl->kc = pl->units >= 2 ? 2 : 1; pl->kc >= 1; --pl->kc) {
    pl->x_off = pl->kc * tile;
    pl->bmin_off = pl->x_off + pl->kc * 4096;
    pl->stage_bytes = pl->bmin_off + pl->kc * 512;
    if (128 + 2 * (size_t)pl->stage_bytes <= half_sm) break;
  }
  if (pl->kc < 1) return false;
  int nst = 4;
  for (; nst >= 2; --nst) {
    pl->smem = 128 + (size_t)nst * pl->stage_bytes;
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

ishi_status ensure_workspace(ishi_ctx *ctx, Workspace *ws, size_t floats, size_t counters) {
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
    ISHI_CUDA(ctx, cudaMemset(ws->counters, 0, counters * sizeof(unsigned int)));
    ws->n_counters = counters;
  }
  return ISHI_OK;
}

template <class Fmt, int MT, int UW>
ishi_status launch_stream(ishi_ctx *ctx, const Plan &pl, const StreamArgs &args, cudaStream_t st) {
  auto kern = stream_kernel<Fmt, MT, UW>;
  static bool configured[64] = {false};  // per device, per kernel instantiation
  static std::mutex once;
  {
    std::lock_guard<std::mutex> g(once);
    if (!configured[ctx->device & 63]) {
      ISHI_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          std::min(kSmemBudget, ctx->smem_optin)));
      configured[ctx->device & 63] = true;
    }
  }
  const int grid = pl.Gc * pl.S;
  const int block = (pl.W + 1) * 32;
  kern<<<grid, block, pl.smem, st>>>(args);
  ISHI_CUDA(ctx, cudaGetLastError());
  return ISHI_OK;
}

template <class Fmt>
ishi_status launch_row(ishi_ctx *ctx, const RowPlan &pl, const RowArgs &args, cudaStream_t st) {
  auto kern = rowstream_kernel<Fmt>;
  static bool configured[64] = {false};
  static std::mutex once;
  {
    std::lock_guard<std::mutex> g(once);
    if (!configured[ctx->device & 63]) {
      ISHI_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (std::min(kSmemBudget, ctx->smem_optin) - 2048) / 2));
      configured[ctx->device & 63] = true;
    }
  }
  kern<<<pl.grid, kRowThreads, pl.smem, st>>>(args);
  ISHI_CUDA(ctx, cudaGetLastError());
  return ISHI_OK;
}

struct GgmlCall {
  const void *x;
  int rows;
  const void *blocks;
  int type;
  long long n, k;
  void *y;
  long long ldy;
  int flags;
};

ishi_status run_ggml_mma(ishi_ctx *ctx, const Plan &pl, Workspace *ws, const GgmlCall &c,
                         cudaStream_t st) {
  StreamArgs a;
  memset(&a, 0, sizeof(a));
  const int ts = type_size(c.type);
  a.src[0].base = static_cast<const uint8_t *>(c.blocks);
  a.src[0].row_bytes = (long long)(c.k / 256) * ts;
  a.src[0].unit_bytes = ts;
  a.src[0].seg_off = 0;
  a.nsrc = 1;
  a.x = static_cast<const __half *>(c.x);
  a.y = static_cast<__half *>(c.y);
  a.ldy = c.ldy;
  a.out_transposed = (c.flags & ISHI_OUT_TRANSPOSED) ? 1 : 0;
  a.scratch = ws->scratch;
  a.counters = ws->counters;
  a.err = ctx->err_dev;
  a.M = c.rows;
  a.N = (int)c.n;
  a.K = (int)c.k;
  a.units = pl.units;
  a.S = pl.S;
  a.P = pl.P;
  a.Gc = pl.Gc;
  a.SL = pl.SL;
  a.W = pl.W;
  a.nstages = pl.nstages;
  a.row_stride = pl.row_stride;
  switch (c.type) {
    case ISHI_GGML_Q4_K:
      return pl.MT == 1 ? launch_stream<FmtQ4K, 1, 2>(ctx, pl, a, st)
                        : launch_stream<FmtQ4K, 2, 1>(ctx, pl, a, st);
    default:
      return fail(ctx, ISHI_E_UNSUPPORTED, "no matmul kernel for GGML type %d", c.type);
  }
}

ishi_status run_row(ishi_ctx *ctx, const RowPlan &pl, Workspace *ws, const uint8_t *tiles, int fmt, const void *x,
                    int rows, long long n, long long k, void *y, long long ldy, int flags, int group_size,
                    int scale_dtype, cudaStream_t st) {
  RowArgs a;
  memset(&a, 0, sizeof(a));
  a.tiles = tiles;
  a.tile_bytes = pl.tile_bytes;
  for (int i = 0; i < kMaxSrc; ++i) {
    a.sec_off[i] = pl.sec_off[i];
    a.unit_bytes[i] = pl.unit_bytes[i];
  }
  a.x = static_cast<const __half *>(x);
  a.y = static_cast<__half *>(y);
  a.ldy = ldy;
  a.out_transposed = (flags & ISHI_OUT_TRANSPOSED) ? 1 : 0;
  a.scratch = ws->scratch;
  a.counters = ws->counters;
  a.err = ctx->err_dev;
  a.M = rows;
  a.N = (int)n;
  a.K = (int)k;
  a.units = pl.units;
  a.P = pl.P;
  a.SL = pl.SL;
  a.kc = pl.kc;
  a.nstages = pl.nstages;
  a.x_off = pl.x_off;
  a.bmin_off = pl.bmin_off;
  a.stage_bytes = pl.stage_bytes;
  a.group_size = group_size;
  a.scale_dtype = scale_dtype;
  switch (fmt) {
    case ISHI_GGML_Q4_K: return launch_row<RowQ4K>(ctx, pl, a, st);
    default: return fail(ctx, ISHI_E_UNSUPPORTED, "no tcgen05 kernel for format %d", fmt);
  }
}

bool has_row_kernel(int fmt) { return fmt == ISHI_GGML_Q4_K; }

ishi_status check_ggml_call(ishi_ctx *ctx, const GgmlCall &c, long long blocks_bytes, int max_rows) {
  if (!ctx) return ISHI_E_INVALID;
  if (!c.x || !c.blocks || !c.y) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (!aligned16(c.x) || !aligned16(c.blocks)) return fail(ctx, ISHI_E_INVALID, "x and blocks must be 16-byte aligned");
  const int ts = type_size(c.type);
  if (ts == 0) return fail(ctx, ISHI_E_UNSUPPORTED, "GGML type %d has no decoder here", c.type);
  if (c.rows < 1 || c.rows > max_rows) return fail(ctx, ISHI_E_SHAPE, "rows %d outside 1...%d", c.rows, max_rows);
  if (c.k <= 0 || c.k % 256 != 0) return fail(ctx, ISHI_E_SHAPE, "k %lld is not a whole number of 256-blocks", c.k);
  if (c.n <= 0) return fail(ctx, ISHI_E_SHAPE, "n must be positive");
  if (c.n > (1ll << 31) - 16 || c.k > (1ll << 30)) return fail(ctx, ISHI_E_SHAPE, "shape too large");
  if (blocks_bytes < c.n * (c.k / 256) * ts) return fail(ctx, ISHI_E_SHAPE, "block buffer shorter than n * k/256 * type size");
  return ISHI_OK;
}

int unit_bytes_ggml(int type) { return type_size(type); }

int row_skew_for(int fmt) {
  switch (fmt) {
    case ISHI_GGML_Q4_K: return FmtQ4K::kRowSkew;
    default: return 32;
  }
}

}  // namespace

// ---------------------------------------------------------------------------------------------

extern "C" {

const char *ishi_status_string(ishi_status s) {
  switch (s) {
    case ISHI_OK: return "ok";
    case ISHI_E_INVALID: return "invalid argument";
    case ISHI_E_SHAPE: return "shape outside the supported range";
    case ISHI_E_UNSUPPORTED: return "unsupported format";
    case ISHI_E_CUDA: return "CUDA error";
    case ISHI_E_TIMEOUT: return "device-side wait timed out";
    case ISHI_E_NOMEM: return "out of memory";
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
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(c_iq2xs_codes, ISHI_IQ2XS_CODES, sizeof(ISHI_IQ2XS_CODES));
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
  if (ctx->ws.scratch) cudaFree(ctx->ws.scratch);
  if (ctx->ws.counters) cudaFree(ctx->ws.counters);
  if (ctx->err_host) cudaFreeHost(ctx->err_host);
  if (ctx->pin_x) cudaFreeHost(ctx->pin_x);
  if (ctx->pin_y) cudaFreeHost(ctx->pin_y);
  if (ctx->dev_x) cudaFree(ctx->dev_x);
  if (ctx->dev_y) cudaFree(ctx->dev_y);
  delete ctx;
}

ishi_status ishi_ctx_poll(ishi_ctx *ctx) {
  if (!ctx) return ISHI_E_INVALID;
  volatile int *flag = ctx->err_host;
  if (*flag != 0) {
    *flag = 0;
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

ishi_status ishi_ggml_dequantize(ishi_ctx *ctx, int type, const void *blocks, int64_t n_blocks,
                                 void *out, int out_dtype, void *stream) {
  if (!ctx) return ISHI_E_INVALID;
  if (!blocks || !out) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (type_size(type) == 0) return fail(ctx, ISHI_E_UNSUPPORTED, "GGML type %d has no decoder here", type);
  if (n_blocks < 0) return fail(ctx, ISHI_E_SHAPE, "negative block count");
  if (n_blocks == 0) return ISHI_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int threads = 256;
  const long long want = (n_blocks * 32 + threads - 1) / threads;
  const int grid = (int)std::min<long long>(want, (long long)ctx->sm_count * 32);
  const uint8_t *b = static_cast<const uint8_t *>(blocks);
#define ISHI_DQ(T, OT) ggml_dequantize_kernel<T, OT><<<grid, threads, 0, st>>>(b, n_blocks, static_cast<OT *>(out))
#define ISHI_DQ_T(T)                                                   \
  switch (out_dtype) {                                                 \
    case ISHI_DT_F32: ISHI_DQ(T, float); break;                        \
    case ISHI_DT_F16: ISHI_DQ(T, __half); break;                       \
    case ISHI_DT_BF16: ISHI_DQ(T, __nv_bfloat16); break;               \
    default: return fail(ctx, ISHI_E_INVALID, "bad output dtype %d", out_dtype); \
  }
  switch (type) {
    case ISHI_GGML_Q4_K: ISHI_DQ_T(12); break;
    case ISHI_GGML_Q6_K: ISHI_DQ_T(14); break;
    default: ISHI_DQ_T(17); break;
  }
#undef ISHI_DQ_T
#undef ISHI_DQ
  ISHI_CUDA(ctx, cudaGetLastError());
  return ISHI_OK;
}

ishi_status ishi_affine_dequantize(ishi_ctx *ctx, const void *w, const void *scales, const void *biases,
                                   int scale_dtype, int group_size, int bits, int64_t n, int64_t k,
                                   float *out, void *stream) {
  if (!ctx) return ISHI_E_INVALID;
  if (!w || !scales || !biases || !out) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (bits < 2 || bits > 8) return fail(ctx, ISHI_E_SHAPE, "bits %d outside 2...8", bits);
  if (scale_dtype < ISHI_DT_F16 || scale_dtype > ISHI_DT_F32) return fail(ctx, ISHI_E_INVALID, "bad scale dtype");
  if (group_size <= 0 || k <= 0 || n <= 0 || k % group_size != 0 || (k * bits) % 32 != 0)
    return fail(ctx, ISHI_E_SHAPE, "k %lld does not fit groups of %d at %d bits", (long long)k, group_size, bits);
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
  const int threads = std::max(32, std::min(256, block / 2));
  hadamard_rotate_kernel<<<(int)grid, threads, block * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half *>(x), width, block, signs, static_cast<__half *>(y));
  ISHI_CUDA(ctx, cudaGetLastError());
  return ISHI_OK;
}

ishi_status ishi_ggml_matmul_few(ishi_ctx *ctx, const void *x, int rows, const void *blocks,
                                 int64_t blocks_bytes, int type, int64_t n, int64_t k, void *y,
                                 void *stream) {
  GgmlCall c{x, rows, blocks, type, n, k, y, n, 0};
  ishi_status s = check_ggml_call(ctx, c, blocks_bytes, 16);
  if (s != ISHI_OK) return s;
  std::lock_guard<std::mutex> g(ctx->lock);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  Plan pl;
  int ub = unit_bytes_ggml(type);
  if (!make_plan(ctx, type, n, k, rows, 1, &ub, row_skew_for(type), &pl))
    return fail(ctx, ISHI_E_SHAPE, "no launch plan fits shared memory for k %lld", (long long)k);
  s = ensure_workspace(ctx, &ctx->ws, pl.scratch_floats, (size_t)pl.P);
  if (s != ISHI_OK) return s;
  return run_ggml_mma(ctx, pl, &ctx->ws, c, static_cast<cudaStream_t>(stream));
}

// ---- projection -------------------------------------------------------------------------------

struct ishi_projection_impl;

ishi_status ishi_ggml_matvec(ishi_ctx *ctx, const void *x, int rows, const void *blocks,
                             int64_t blocks_bytes, int type, int64_t n, int64_t k, void *y,
                             void *stream) {
  (void)x; (void)rows; (void)blocks; (void)blocks_bytes; (void)type; (void)n; (void)k; (void)y; (void)stream;
  return fail(ctx, ISHI_E_UNSUPPORTED, "matvec kernel not built yet");
}

ishi_status ishi_verify_matmul(ishi_ctx *ctx, const void *, int, const void *, const void *, const void *,
                               int, int, int, int64_t, int64_t, int, void *, void *) {
  return fail(ctx, ISHI_E_UNSUPPORTED, "affine kernel not built yet");
}

}  // extern "C"

// ---- projection: the PackedLinear counterpart -----------------------------------------------

struct ishi_projection {
  ishi_ctx *ctx = nullptr;
  ishi_weight_desc d;
  Plan plan[2];       // warp-level kernel: rows 1..8 and rows 9..16
  RowPlan row;        // tcgen05 kernel: rows 1..8
  uint8_t *tiles = nullptr;  // the weight re-tiled for the tcgen05 kernel (library-owned)
  int fmt = 0;
  Workspace ws;       // this projection's own scratch, so apply never allocates
  __half *xr = nullptr;  // rotated activations [16][k] when the pack is rotated
  int64_t weight_bytes = 0;
};

namespace {

ishi_status projection_matmul(ishi_projection *p, const void *x, int rows, void *y, int64_t ldy,
                              int flags, cudaStream_t st) {
  ishi_ctx *ctx = p->ctx;
  if (!x || !y) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (!aligned16(x)) return fail(ctx, ISHI_E_INVALID, "x must be 16-byte aligned");
  if (rows < 1 || rows > 16) return fail(ctx, ISHI_E_SHAPE, "rows %d outside 1...16", rows);
  const int64_t need_ld = (flags & ISHI_OUT_TRANSPOSED) ? rows : p->d.n;
  if (ldy < need_ld) return fail(ctx, ISHI_E_SHAPE, "ldy %lld shorter than %lld", (long long)ldy, (long long)need_ld);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  const Plan &pl = p->plan[rows > 8 ? 1 : 0];
  if (p->d.kind == ISHI_KIND_GGML) {
    GgmlCall c{x, rows, p->d.weight_dev, p->d.ggml_type, p->d.n, p->d.k, y, ldy, flags};
    if (rows <= 8 && p->row.ok && ctx->route != ISHI_ROUTE_GEMV)
      return run_row(ctx, p->row, &p->ws, p->tiles, p->fmt, x, rows, p->d.n, p->d.k, y, ldy, flags, 0, 0, st);
    return run_ggml_mma(ctx, pl, &p->ws, c, st);
  }
  return fail(ctx, ISHI_E_UNSUPPORTED, "affine kernel not built yet");
}

}  // namespace

extern "C" {

ishi_status ishi_projection_create(ishi_ctx *ctx, const ishi_weight_desc *desc, ishi_projection **out) {
  if (!ctx || !out) return ISHI_E_INVALID;
  *out = nullptr;
  if (!desc) return fail(ctx, ISHI_E_INVALID, "null descriptor");
  const ishi_weight_desc &d = *desc;
  if (!d.weight_dev || !aligned16(d.weight_dev)) return fail(ctx, ISHI_E_INVALID, "weight pointer null or not 16-byte aligned");
  if (d.n <= 0 || d.k <= 0) return fail(ctx, ISHI_E_SHAPE, "n and k must be positive");
  if (d.n > (1ll << 31) - 16 || d.k > (1ll << 30)) return fail(ctx, ISHI_E_SHAPE, "shape too large");
  if (d.k % 256 != 0) return fail(ctx, ISHI_E_SHAPE, "k %lld is not a multiple of 256", (long long)d.k);
  if (d.hadamard_block != 0) {
    const int b = d.hadamard_block;
    if (b < 0 || (b & (b - 1)) != 0 || b > 8192 || d.k % b != 0)
      return fail(ctx, ISHI_E_SHAPE, "Hadamard block %d does not divide input width %lld", b, (long long)d.k);
  }
  int nsrc = 0, unit_bytes[kMaxSrc] = {0, 0, 0}, fmt = 0;
  int64_t bytes = 0;
  if (d.kind == ISHI_KIND_GGML) {
    const int ts = type_size(d.ggml_type);
    if (ts == 0) return fail(ctx, ISHI_E_UNSUPPORTED, "GGML type %d has no decoder here", d.ggml_type);
    bytes = d.n * (d.k / 256) * ts;
    nsrc = 1;
    unit_bytes[0] = ts;
    fmt = d.ggml_type;
  } else if (d.kind == ISHI_KIND_AFFINE) {
    if (d.bits != 2 && d.bits != 4 && d.bits != 8) return fail(ctx, ISHI_E_UNSUPPORTED, "affine width %d has no kernel here", d.bits);
    if (d.group_size != 32 && d.group_size != 64 && d.group_size != 128) return fail(ctx, ISHI_E_SHAPE, "group size %d outside {32, 64, 128}", d.group_size);
    if (d.scale_dtype < ISHI_DT_F16 || d.scale_dtype > ISHI_DT_F32) return fail(ctx, ISHI_E_INVALID, "bad scale dtype");
    if (!d.scales_dev || !d.biases_dev || !aligned16(d.scales_dev) || !aligned16(d.biases_dev))
      return fail(ctx, ISHI_E_INVALID, "scales/biases null or not 16-byte aligned");
    const int sb = d.scale_dtype == ISHI_DT_F32 ? 4 : 2;
    bytes = d.n * d.k * d.bits / 8;
    nsrc = 3;
    unit_bytes[0] = 256 * d.bits / 8;
    unit_bytes[1] = unit_bytes[2] = 256 / d.group_size * sb;
    fmt = 100 + d.bits;
  } else {
    return fail(ctx, ISHI_E_INVALID, "bad weight kind %d", d.kind);
  }
  if (d.weight_bytes < bytes) return fail(ctx, ISHI_E_SHAPE, "weight buffer holds %lld bytes, shape needs %lld", (long long)d.weight_bytes, (long long)bytes);

  std::lock_guard<std::mutex> g(ctx->lock);
  ISHI_CUDA(ctx, cudaSetDevice(ctx->device));
  ishi_projection *p = new (std::nothrow) ishi_projection();
  if (!p) return fail(ctx, ISHI_E_NOMEM, "out of host memory");
  p->ctx = ctx;
  p->d = d;
  p->weight_bytes = bytes;
  if (d.kind == ISHI_KIND_AFFINE) {
    const int sb = d.scale_dtype == ISHI_DT_F32 ? 4 : 2;
    p->weight_bytes += 2 * d.n * (d.k / d.group_size) * sb;
  }
  size_t floats = 0;
  for (int i = 0; i < 2; ++i) {
    if (!make_plan(ctx, fmt, d.n, d.k, i ? 16 : 8, nsrc, unit_bytes, row_skew_for(fmt), &p->plan[i])) {
      delete p;
      return fail(ctx, ISHI_E_SHAPE, "no launch plan fits shared memory for k %lld", (long long)d.k);
    }
    floats = std::max(floats, p->plan[i].scratch_floats);
  }
  size_t counters = (size_t)p->plan[0].P;
  p->fmt = fmt;
  if (has_row_kernel(fmt) && make_row_plan(ctx, d.n, d.k, nsrc, unit_bytes, &p->row)) {
    floats = std::max(floats, p->row.scratch_floats);
    counters = std::max(counters, p->row.counters);
  }
  ishi_status s = ensure_workspace(ctx, &p->ws, floats, counters);
  if (s == ISHI_OK && p->row.ok) {
    // re-tile the weight once; the caller's buffer stays as it is and is still used for 9...16 rows
    cudaError_t e = cudaMalloc(&p->tiles, p->row.tiles_bytes);
    if (e != cudaSuccess) {
      s = fail(ctx, ISHI_E_CUDA, "cudaMalloc(tiled weight, %zu bytes): %s", p->row.tiles_bytes, cudaGetErrorString(e));
    } else {
      TileSrc ts[kMaxSrc];
      memset(ts, 0, sizeof(ts));
      const void *bases[kMaxSrc] = {d.weight_dev, d.scales_dev, d.biases_dev};
      for (int i = 0; i < nsrc; ++i) {
        ts[i].base = static_cast<const uint8_t *>(bases[i]);
        ts[i].unit_bytes = unit_bytes[i];
        ts[i].row_bytes = (long long)(d.k / 256) * unit_bytes[i];
        ts[i].sec_off = p->row.sec_off[i];
      }
      const long long triples = (long long)p->row.P * p->row.units * kRowPanel;
      const int grid = (int)std::min<long long>((triples + 255) / 256, (long long)ctx->sm_count * 16);
      prepare_tiles_kernel<<<grid, 256>>>(ts[0], ts[1], ts[2], nsrc, d.n, p->row.units, p->row.tile_bytes, p->tiles);
      e = cudaGetLastError();
      if (e == cudaSuccess) e = cudaDeviceSynchronize();
      if (e != cudaSuccess) s = fail(ctx, ISHI_E_CUDA, "tiling the weight: %s", cudaGetErrorString(e));
    }
  }
  if (s == ISHI_OK && d.hadamard_block != 0) {
    cudaError_t e = cudaMalloc(&p->xr, (size_t)16 * d.k * sizeof(__half));
    if (e != cudaSuccess) s = fail(ctx, ISHI_E_CUDA, "cudaMalloc(rotated x): %s", cudaGetErrorString(e));
  }
  if (s != ISHI_OK) {
    ishi_projection_destroy(p);
    return s;
  }
  *out = p;
  return ISHI_OK;
}

void ishi_projection_destroy(ishi_projection *p) {
  if (!p) return;
  cudaSetDevice(p->ctx->device);
  if (p->ws.scratch) cudaFree(p->ws.scratch);
  if (p->ws.counters) cudaFree(p->ws.counters);
  if (p->xr) cudaFree(p->xr);
  if (p->tiles) cudaFree(p->tiles);
  delete p;
}

int64_t ishi_projection_input_dim(const ishi_projection *p) { return p ? p->d.k : 0; }
int64_t ishi_projection_output_dim(const ishi_projection *p) { return p ? p->d.n : 0; }
int64_t ishi_projection_weight_bytes(const ishi_projection *p) { return p ? p->weight_bytes : 0; }
int ishi_projection_crossover_rows(const ishi_projection *p) {
  if (!p) return 0;
  return p->ctx->crossover_rows > 0 ? p->ctx->crossover_rows : 1;
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
  return projection_matmul(p, xr, rows, y, ldy, flags, static_cast<cudaStream_t>(stream));
}

ishi_status ishi_projection_apply(ishi_projection *p, const void *x, int rows, void *y, int64_t ldy, int flags,
                                  void *stream) {
  if (!p) return ISHI_E_INVALID;
  if (p->d.hadamard_block == 0) return projection_matmul(p, x, rows, y, ldy, flags, static_cast<cudaStream_t>(stream));
  if (rows < 1 || rows > 16) return fail(p->ctx, ISHI_E_SHAPE, "rows %d outside 1...16", rows);
  ishi_status s = ishi_projection_rotate(p, x, rows, p->xr, stream);
  if (s != ISHI_OK) return s;
  return projection_matmul(p, p->xr, rows, y, ldy, flags, static_cast<cudaStream_t>(stream));
}

ishi_status ishi_projection_apply_host(ishi_projection *p, const void *x_host, int rows, void *y_host, void *stream) {
  if (!p) return ISHI_E_INVALID;
  ishi_ctx *ctx = p->ctx;
  if (!x_host || !y_host) return fail(ctx, ISHI_E_INVALID, "null pointer");
  if (rows < 1 || rows > 16) return fail(ctx, ISHI_E_SHAPE, "rows %d outside 1...16", rows);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t xb = (size_t)rows * p->d.k * sizeof(__half), yb = (size_t)rows * p->d.n * sizeof(__half);
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
      const size_t cap = (size_t)16 * p->d.n * sizeof(__half);
      ISHI_CUDA(ctx, cudaHostAlloc(&ctx->pin_y, cap, cudaHostAllocDefault));
      ISHI_CUDA(ctx, cudaMalloc(&ctx->dev_y, cap));
      ctx->pin_y_bytes = cap;
    }
  }
  memcpy(ctx->pin_x, x_host, xb);
  ISHI_CUDA(ctx, cudaMemcpyAsync(ctx->dev_x, ctx->pin_x, xb, cudaMemcpyHostToDevice, st));
  ishi_status s = ishi_projection_apply(p, ctx->dev_x, rows, ctx->dev_y, p->d.n, 0, stream);
  if (s != ISHI_OK) return s;
  ISHI_CUDA(ctx, cudaMemcpyAsync(ctx->pin_y, ctx->dev_y, yb, cudaMemcpyDeviceToHost, st));
  ISHI_CUDA(ctx, cudaStreamSynchronize(st));
  memcpy(y_host, ctx->pin_y, yb);
  return ishi_ctx_poll(ctx);
}

}  // extern "C"
