// N-sharded projections assembled with one NCCL all-gather per projection, behind the C ABI.
//
// NCCL is not linked: it is looked up at run time (dlopen of libnccl.so.2, which resolves to the
// copy a host process has already loaded, if any), so that a single-GPU host needs no NCCL at
// all. The communicator is created in NCCL's non-blocking mode and every call that may still be
// in progress is polled with ncclCommGetAsyncError against a host-side time limit: a peer that
// never shows up ends in ISHI_E_TIMEOUT and an aborted communicator, not in a hung process.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <thread>

#include "../../include/ishizuki_cuda.h"

namespace {

// the part of NCCL this file uses; a test can put its own functions here (ishi_group_debug_set_api)
struct NcclApi {
  ncclResult_t (*get_unique_id)(ncclUniqueId *);
  ncclResult_t (*comm_init_rank_config)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *);
  ncclResult_t (*comm_get_async_error)(ncclComm_t, ncclResult_t *);
  ncclResult_t (*all_gather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*comm_abort)(ncclComm_t);
  ncclResult_t (*comm_destroy)(ncclComm_t);
  const char *(*get_error_string)(ncclResult_t);
};

NcclApi g_api;
bool g_api_ready = false, g_api_injected = false;
std::mutex g_api_lock;

bool load_api() {
  std::lock_guard<std::mutex> g(g_api_lock);
  if (g_api_ready) return true;
  void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return false;
#define ISHI_SYM(field, name)                                          \
  g_api.field = reinterpret_cast<decltype(g_api.field)>(dlsym(h, name)); \
  if (!g_api.field) return false;
  ISHI_SYM(get_unique_id, "ncclGetUniqueId")
  ISHI_SYM(comm_init_rank_config, "ncclCommInitRankConfig")
  ISHI_SYM(comm_get_async_error, "ncclCommGetAsyncError")
  ISHI_SYM(all_gather, "ncclAllGather")
  ISHI_SYM(comm_abort, "ncclCommAbort")
  ISHI_SYM(comm_destroy, "ncclCommDestroy")
  ISHI_SYM(get_error_string, "ncclGetErrorString")
#undef ISHI_SYM
  g_api_ready = true;
  return true;
}

}  // namespace

struct ishi_group {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1, timeout_ms = 0;
  bool broken = false;
  char last_error[256] = {0};
};

namespace {

ishi_status group_fail(ishi_group *g, ishi_status s, const char *fmt, ...) {
  if (g) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g->last_error, sizeof(g->last_error), fmt, ap);
    va_end(ap);
  }
  return s;
}

// Waits until the communicator's pending operation has been taken over by NCCL, polling its
// asynchronous state; after the time limit the communicator is aborted.
ishi_status settle(ishi_group *g, ncclResult_t first, const char *what) {
  ncclResult_t state = first;
  const auto t0 = std::chrono::steady_clock::now();
  unsigned polls = 0;
  while (state == ncclInProgress) {
    const ncclResult_t q = g_api.comm_get_async_error(g->comm, &state);
    if (q != ncclSuccess) {
      state = q;
      break;
    }
    if (state != ncclInProgress) break;
    const auto waited = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
    if (waited > g->timeout_ms) {
      g->broken = true;
      if (g->comm) g_api.comm_abort(g->comm);
      g->comm = nullptr;
      return group_fail(g, ISHI_E_TIMEOUT, "%s: no answer from the other ranks within %d ms; communicator aborted", what,
                        g->timeout_ms);
    }
    if (++polls > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50));  // spin first: it is usually quick
  }
  if (state != ncclSuccess) {
    g->broken = true;
    return group_fail(g, ISHI_E_NCCL, "%s: %s", what, g_api.get_error_string(state));
  }
  return ISHI_OK;
}

}  // namespace

extern "C" {

ishi_status ishi_group_debug_set_api(const void *table) {
  std::lock_guard<std::mutex> g(g_api_lock);
  if (!table) {
    g_api_ready = g_api_injected = false;
    return ISHI_OK;
  }
  memcpy(&g_api, table, sizeof(g_api));
  g_api_ready = g_api_injected = true;
  return ISHI_OK;
}

ishi_status ishi_group_unique_id(void *id_out) {
  if (!id_out) return ISHI_E_INVALID;
  if (!load_api()) return ISHI_E_UNSUPPORTED;
  static_assert(sizeof(ncclUniqueId) <= ISHI_GROUP_ID_BYTES, "the id fits the exported blob");
  ncclUniqueId id;
  memset(&id, 0, sizeof(id));
  if (g_api.get_unique_id(&id) != ncclSuccess) return ISHI_E_NCCL;
  memset(id_out, 0, ISHI_GROUP_ID_BYTES);
  memcpy(id_out, &id, sizeof(id));
  return ISHI_OK;
}

ishi_status ishi_group_create(const void *id_bytes, int rank, int world, int timeout_ms, ishi_group **out) {
  if (!out) return ISHI_E_INVALID;
  *out = nullptr;
  if (!id_bytes || world < 1 || world > 8 || rank < 0 || rank >= world || timeout_ms <= 0) return ISHI_E_INVALID;
  if (!load_api()) return ISHI_E_UNSUPPORTED;
  ishi_group *g = new (std::nothrow) ishi_group();
  if (!g) return ISHI_E_NOMEM;
  g->rank = rank;
  g->world = world;
  g->timeout_ms = timeout_ms;
  ncclUniqueId id;
  memcpy(&id, id_bytes, sizeof(id));
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  cfg.blocking = 0;
  ncclResult_t r = g_api.comm_init_rank_config(&g->comm, world, id, rank, &cfg);
  if (r != ncclSuccess && r != ncclInProgress) {
    group_fail(g, ISHI_E_NCCL, "ncclCommInitRankConfig: %s", g_api.get_error_string(r));
    *out = g;  // kept so that the caller can read the message; destroy it as usual
    g->broken = true;
    return ISHI_E_NCCL;
  }
  const ishi_status s = settle(g, ncclInProgress, "creating the communicator");
  *out = g;
  return s;
}

const char *ishi_group_last_error(const ishi_group *g) { return g ? g->last_error : "null group"; }

ishi_status ishi_projection_apply_sharded(ishi_group *g, ishi_projection *p, const void *x_dev, int rows, void *y_all_dev,
                                          void *stream) {
  if (!g || !p) return ISHI_E_INVALID;
  if (g->broken || !g->comm) return group_fail(g, ISHI_E_NCCL, "the communicator is no longer usable");
  if (!x_dev || !y_all_dev) return group_fail(g, ISHI_E_INVALID, "null pointer");
  if (rows < 1 || rows > 16) return group_fail(g, ISHI_E_SHAPE, "rows %d outside 1...16", rows);
  // The collective is enqueued eagerly only: inside a stream capture the communicator's host-side
  // progress (connection setup, asynchronous error polling) is not ordered by the graph.
  if (g->world > 1) {
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &capturing) != cudaSuccess) {
      cudaGetLastError();
      return group_fail(g, ISHI_E_CUDA, "cudaStreamIsCapturing failed");
    }
    if (capturing != cudaStreamCaptureStatusNone)
      return group_fail(g, ISHI_E_UNSUPPORTED, "the sharded product with an all-gather cannot be captured in a CUDA graph");
  }
  const int64_t n_local = ishi_projection_output_dim(p);
  // this rank's rows, transposed, straight into its slab of the gathered array
  __half *slab = static_cast<__half *>(y_all_dev) + (size_t)g->rank * n_local * rows;
  ishi_status s = ishi_projection_apply(p, x_dev, rows, slab, rows, ISHI_OUT_TRANSPOSED, stream);
  if (s != ISHI_OK) return s;
  if (g->world == 1) return ISHI_OK;
  const ncclResult_t r = g_api.all_gather(slab, y_all_dev, (size_t)n_local * rows, ncclHalf, g->comm,
                                          static_cast<cudaStream_t>(stream));
  if (r != ncclSuccess && r != ncclInProgress) {
    g->broken = true;
    return group_fail(g, ISHI_E_NCCL, "ncclAllGather: %s", g_api.get_error_string(r));
  }
  return settle(g, ncclInProgress, "enqueueing the all-gather");
}

void ishi_group_destroy(ishi_group *g) {
  if (!g) return;
  if (g->comm && g_api_ready) {
    if (g->broken) g_api.comm_abort(g->comm);
    else g_api.comm_destroy(g->comm);
  }
  delete g;
}

}  // extern "C"
