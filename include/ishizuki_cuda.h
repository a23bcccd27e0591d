/* C ABI of the B200 verify-matmul library (libishizuki_cuda.so).
 *
 * This is the boundary a host binding (Swift over a SwiftPM C target, or ctypes) links against.
 * It replaces, for NVIDIA B200, the kernel layer the reference reaches through
 * MLXFast.metalKernel: each entry point names the reference interface it stands in for, by the
 * file's path inside the reference project.
 *
 * Conventions
 *   - Every pointer named *_dev is a device pointer on the context's GPU; the caller owns every
 *     buffer it passes. ishi_projection_create COPIES the weight into the library's own tiled
 *     layout (same bytes, same compression, another order) and never reads the caller's buffer
 *     again: the caller may free it after create, and until it does the weight is held twice.
 *     The kernel-level calls (ishi_ggml_matvec, ishi_ggml_matmul_few, ishi_verify_matmul) take a
 *     raw weight and re-tile it into the context's scratch on EVERY call (they may reallocate
 *     that scratch): they exist for tests and tools, a decode loop uses projections.
 *   - Activations are fp16 row-major [M, K]; outputs are fp16 [M, N] with leading dimension
 *     ldy (elements), or [N, M] with leading dimension ldy when ISHI_OUT_TRANSPOSED is set.
 *     Accumulation is fp32.
 *   - Calls are asynchronous on the given CUDA stream (a cudaStream_t passed as void*; NULL is
 *     the default stream). Calls that share a context or a projection share its scratch memory
 *     and must be ordered on one stream (or otherwise not overlap on the GPU).
 *   - Every function returns an ishi_status and never aborts the process. Where the reference
 *     returns nil ("this shape is declined, fall back"), this library returns
 *     ISHI_E_UNSUPPORTED or ISHI_E_SHAPE: there is no CPU or library fallback behind it.
 */
#ifndef ISHIZUKI_CUDA_H
#define ISHIZUKI_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int ishi_status;
enum {
  ISHI_OK = 0,
  ISHI_E_INVALID = 1,     /* null or misaligned pointer, bad enum value */
  ISHI_E_SHAPE = 2,       /* a shape guard of the reference failed (K % 256, rows out of range ...) */
  ISHI_E_UNSUPPORTED = 3, /* a format or width this library has no kernel for */
  ISHI_E_CUDA = 4,        /* a CUDA runtime call failed; see ishi_last_error */
  ISHI_E_TIMEOUT = 5,     /* a bounded device-side wait gave up; outputs of that call are invalid */
  ISHI_E_NOMEM = 6,
  ISHI_E_TOO_LARGE = 7,   /* larger than the built-in scratch of ishi_q4k_matmul_few_static */
  ISHI_E_NCCL = 8         /* an NCCL call failed or the communicator was aborted; see ishi_group_last_error */
};

/* GGML block types, numbered as in GGUF (Sources/IshizukiKit/Config/GGUFFile.swift:13-44): the
 * eleven quantized types the reference reads (GGMLDequant.supported,
 * Sources/IshizukiKit/Core/GGMLDequant.swift:19-24). Every one of them has a fragment decoder on
 * the warp-level product kernel (the weight is decoded inside the multiply, never expanded in
 * memory); a one-warp-per-row kernel on the plain blocks is the fallback for inputs too wide for it. */
enum {
  ISHI_GGML_Q2_K = 10, ISHI_GGML_Q4_K = 12, ISHI_GGML_Q6_K = 14, ISHI_GGML_IQ2_XXS = 16, ISHI_GGML_IQ2_XS = 17,
  ISHI_GGML_IQ3_XXS = 18, ISHI_GGML_IQ1_S = 19, ISHI_GGML_IQ3_S = 21, ISHI_GGML_IQ2_S = 22, ISHI_GGML_IQ4_XS = 23,
  ISHI_GGML_IQ1_M = 29
};

enum { ISHI_KIND_AFFINE = 0, ISHI_KIND_GGML = 1 };
enum { ISHI_DT_F16 = 0, ISHI_DT_BF16 = 1, ISHI_DT_F32 = 2 };

/* Which kernel family a call uses. AUTO applies the per-projection row-count crossover. */
enum { ISHI_ROUTE_AUTO = 0, ISHI_ROUTE_GEMV = 1, ISHI_ROUTE_MMA = 2 };

enum { ISHI_OUT_TRANSPOSED = 1 };

typedef struct ishi_ctx ishi_ctx;
typedef struct ishi_projection ishi_projection;

/* One projection's weight, as PackedLinear's initialisers receive it
 * (Sources/IshizukiKit/Core/Hadamard.swift:51-86 for affine packs, :110-124 for GGUF blocks).
 * n is the number of output rows held by THIS weight buffer: an N-shard passes its own rows. */
typedef struct ishi_weight_desc {
  int32_t kind;           /* ISHI_KIND_* */
  int32_t ggml_type;      /* ISHI_GGML_* when kind == GGML */
  int32_t bits;           /* affine: 2, 4 or 8 */
  int32_t group_size;     /* affine: 32, 64 or 128 */
  int32_t scale_dtype;    /* affine: ISHI_DT_* of scales and biases */
  int32_t hadamard_block; /* 0, or the power-of-two block of the input rotation */
  int64_t n;              /* output rows in this buffer */
  int64_t k;              /* input width */
  const void *weight_dev; /* GGUF: raw blocks [n][k/256][type size]; affine: uint32 [n][k*bits/32] */
  int64_t weight_bytes;   /* size of weight_dev, checked against the shape */
  const void *scales_dev; /* affine: [n][k/group_size] */
  const void *biases_dev; /* affine: [n][k/group_size] */
  const float *signs_dev; /* rotation signs [k] of +-1, or NULL for none */
} ishi_weight_desc;

/* ---- context ------------------------------------------------------------------------------ */

/* One context per GPU and per stream of work. Allocates the library's tables and scratch. */
ishi_status ishi_ctx_create(int device, ishi_ctx **out);
void ishi_ctx_destroy(ishi_ctx *ctx);
const char *ishi_status_string(ishi_status s);
/* Text of the last failure seen through this context (valid until the next call). */
const char *ishi_last_error(const ishi_ctx *ctx);
/* Returns ISHI_E_TIMEOUT if any kernel launched through this context has reported that a
 * bounded wait gave up since the last poll, else ISHI_OK. Does not synchronise. */
ishi_status ishi_ctx_poll(ishi_ctx *ctx);
/* Runtime switches, the counterpart of BonsaiRuntime.useVerifyMatmul and the tunables of
 * VerifyMatmul (Sources/IshizukiKit/Core/RuntimeOptions.swift:43-54,
 * Sources/IshizukiKit/Core/VerifyMatmul.swift:28-33). route: ISHI_ROUTE_GEMV sends a single row to
 * the CUDA-core kernel (formats of the warp-level kernel), ISHI_ROUTE_MMA never does, and
 * ISHI_ROUTE_AUTO does when crossover_rows > 1: crossover_rows is the row count from which AUTO
 * uses the tensor-core kernel (0 restores the built-in value, 1: the tensor-core kernel measured
 * faster on B200 at one row on every benchmark shape). */
ishi_status ishi_ctx_set_route(ishi_ctx *ctx, int route, int crossover_rows);

/* ---- projection: PackedLinear ------------------------------------------------------------- */

/* PackedLinear.init + VerifyMatmul.warm (Hadamard.swift:51-86, VerifyMatmul.swift:40-61):
 * validates the weight, allocates the projection's own memory, copies the weight into it in tiled
 * order and fixes the launch plan for its shape: for the warp-level kernel's formats by timing the
 * best few candidate plans on the tiled weight (about a millisecond; ISHI_NO_AUTOTUNE=1 in the
 * environment keeps the estimate's choice). Synchronises the device. */
ishi_status ishi_projection_create(ishi_ctx *ctx, const ishi_weight_desc *desc,
                                   ishi_projection **out);
/* Several weights of one format and input width as ONE projection: their output rows stacked in
 * the order given, y = [x . W0^T | x . W1^T | ...] ([rows, n0 + n1 + ...]). For projections that
 * read the same input (the reference's q/k/v, Sources/IshizukiKit/Text/Attention.swift:75-83, and
 * gate/up, Attention.swift:251, which it runs as separate kernels): one launch streams all of them,
 * so the per-launch costs are paid once. count in 1...4; all descriptors must agree in kind, type,
 * width, group size, scale dtype, k and rotation. Every GGUF block type and the 4-/2-bit affine
 * packs with fp16 / bf16 scales: the formats of the warp-level kernel (ISHI_E_UNSUPPORTED otherwise). */
ishi_status ishi_projection_create_fused(ishi_ctx *ctx, const ishi_weight_desc *descs, int count,
                                         ishi_projection **out);
/* The MLP's gate and up projections as ONE projection whose output is the input of downProj:
 * y = silu(x . gate^T) * (x . up^T), [rows, n] with n the height of either weight
 * (Sources/IshizukiKit/Text/Attention.swift:251, where the reference runs two projections and two
 * element-wise kernels). The rows of the two weights are interleaved by eights in the tiled copy,
 * so one accumulator fragment of the kernel holds a gate row and its up row and the epilogue
 * combines them: no [rows, 2 n] intermediate is written. Roundings as on the reference's fp16
 * arrays: both products, the sigmoid, gate * sigmoid and the final product are each rounded to
 * fp16, the arithmetic is fp32. Same formats as ishi_projection_create_fused; both descriptors
 * must agree as there, n the same for both and a multiple of 8 (ISHI_E_SHAPE otherwise).
 * ishi_projection_output_dim returns n, ishi_projection_weight_bytes the bytes of both weights. */
ishi_status ishi_projection_create_gated(ishi_ctx *ctx, const ishi_weight_desc *gate,
                                         const ishi_weight_desc *up, ishi_projection **out);
void ishi_projection_destroy(ishi_projection *p);
int64_t ishi_projection_input_dim(const ishi_projection *p);  /* Projection.inputDim */
int64_t ishi_projection_output_dim(const ishi_projection *p); /* Projection.outputDim */
/* Compressed weight bytes one apply streams (codes + scales + biases, or GGUF blocks). */
int64_t ishi_projection_weight_bytes(const ishi_projection *p);
/* Rows from which this projection's AUTO route uses the tensor-core kernel: the context's
 * crossover_rows, or the built-in 1. The counterpart of VerifyMatmul.minimumRows(bytes:)
 * (VerifyMatmul.swift:19-26), whose table was tuned for Apple M1 (ishi_reference_minimum_rows). */
int ishi_projection_crossover_rows(const ishi_projection *p);
/* The launch plan create settled on, for the warp-level kernel's formats: {K split = cluster size,
 * warps per panel, panels in parallel, tiles per warp ring} (zeros for the other kernels), and a way
 * to impose one: the order in which partial sums are added follows the plan, so two projections of
 * the same weight agree bit for bit only under the same plan (the tiled copy does not depend on
 * it). set_plan accepts what ishi_projection_plan of a projection of the same shape returned. */
ishi_status ishi_projection_plan(const ishi_projection *p, int plan[4]);
ishi_status ishi_projection_set_plan(ishi_projection *p, const int plan[4]);

/* PackedLinear.callAsFunction (Hadamard.swift:180-213): rotates x when the pack is rotated,
 * then multiplies. rows in 1...16. */
ishi_status ishi_projection_apply(ishi_projection *p, const void *x_dev, int rows, void *y_dev,
                                  int64_t ldy, int flags, void *stream);
/* PackedLinear.rotate (Hadamard.swift:235-243): xr = WHT_block(x * signs) / sqrt(block), fp16.
 * Copies x when the projection has no rotation. */
ishi_status ishi_projection_rotate(ishi_projection *p, const void *x_dev, int rows, void *xr_dev,
                                   void *stream);
/* PackedLinear.applyRotated (Hadamard.swift:245-252): multiplies an already rotated input. */
ishi_status ishi_projection_apply_rotated(ishi_projection *p, const void *xr_dev, int rows,
                                          void *y_dev, int64_t ldy, int flags, void *stream);
/* The language-model head of a greedy verify step: logits = x . W^T, then per row the index of the
 * largest logit (fp16 values, the lowest index among equals, as MLX argMax), which is all the
 * reference's verify loop reads of them (Sources/IshizukiKit/Text/TextModel.swift:350-355,
 * Sources/IshizukiKit/Generate/SpeculativeGeneration.swift:173-177). argmax_dev: int32 [rows]. The
 * logits stay in a buffer the projection owns (allocated by the first call: make it outside
 * stream capture). */
ishi_status ishi_projection_apply_argmax(ishi_projection *p, const void *x_dev, int rows,
                                         int32_t *argmax_dev, void *stream);
/* The same product for a caller whose activations live in host memory: copies x in, multiplies,
 * copies y out, all on the stream; returns once y_host is complete. */
ishi_status ishi_projection_apply_host(ishi_projection *p, const void *x_host, int rows,
                                       void *y_host, void *stream);
/* The same without the wait: enqueues the copy of x_host [rows, k] to the device, the product and
 * the copy of y [rows, n] back into y_host on the stream and returns. Both host buffers must stay
 * untouched until the stream has been synchronised; with page-locked host memory the copies
 * overlap the host, with pageable memory the runtime stages them. Calls on one projection must
 * be ordered on one stream (they share its device staging, allocated by the first call). Errors a
 * kernel raises show in ishi_ctx_poll after the synchronisation. */
ishi_status ishi_projection_apply_host_async(ishi_projection *p, const void *x_host, int rows,
                                             void *y_host, void *stream);

/* A list of projections in one call, each with its own host input x_hosts[i] [rows, k_i] and host
 * output y_hosts[i] [rows, n_i] (page-locked buffers for the copies to overlap): the x copies, the
 * products and the y copies are pipelined over three streams in chunks of sixteen entries, and the
 * caller's stream ends behind all of them, so one cudaStreamSynchronize(stream) completes the whole
 * list. The projections
 * must share a context and are independent of each other (none reads another's output). */
ishi_status ishi_projection_apply_host_batch(ishi_projection *const *projections,
                                             const void *const *x_hosts, int rows,
                                             void *const *y_hosts, int count, void *stream);

/* ---- kernel level ------------------------------------------------------------------------- */

/* GGMLKernels.matvec (Sources/IshizukiKit/Core/GGMLKernels.swift:177-213): x [rows, k] against
 * the blocks of w [n, k]. A single row of a format the warp-level kernel decodes (Q4_K) runs on
 * CUDA cores (fp32 FMA, warp-shuffle reduction); more rows, and the other formats, run the
 * tensor-core kernel, which is the faster one on this GPU at every row count. rows in 1...16. */
ishi_status ishi_ggml_matvec(ishi_ctx *ctx, const void *x_dev, int rows, const void *blocks_dev,
                             int64_t blocks_bytes, int ggml_type, int64_t n, int64_t k,
                             void *y_dev, void *stream);
/* GGMLKernels.matmulFew (GGMLKernels.swift:219-253): the same product with each weight decoded
 * once into a tensor-core fragment. The reference takes rows in 2...8; this takes 1...16. */
ishi_status ishi_ggml_matmul_few(ishi_ctx *ctx, const void *x_dev, int rows,
                                 const void *blocks_dev, int64_t blocks_bytes, int ggml_type,
                                 int64_t n, int64_t k, void *y_dev, void *stream);
/* GGMLKernels.dequantize (GGMLKernels.swift:60-95): blocks to a dense array, bit-exact to
 * ggml's to_float. out_dtype ISHI_DT_F32, ISHI_DT_F16 or ISHI_DT_BF16. */
ishi_status ishi_ggml_dequantize(ishi_ctx *ctx, int ggml_type, const void *blocks_dev,
                                 int64_t n_blocks, void *out_dev, int out_dtype, void *stream);
/* GGMLKernels.gather (GGMLKernels.swift:102-138): rows of a quantized table [table_rows, k] by id,
 * decoded into out [count, k] (the embedding lookup). ids_dev: int32 [count]; an id outside the
 * table gives a row of zeros. */
ishi_status ishi_ggml_gather(ishi_ctx *ctx, const int32_t *ids_dev, int64_t count, const void *blocks_dev,
                             int64_t blocks_bytes, int ggml_type, int64_t table_rows, int64_t k,
                             void *out_dev, int out_dtype, void *stream);
/* VerifyMatmul.applyAny (Sources/IshizukiKit/Core/VerifyMatmul.swift:73-120): x [rows, k]
 * against an affine pack. route picks the kernel (ISHI_ROUTE_GEMV or ISHI_ROUTE_MMA). */
ishi_status ishi_verify_matmul(ishi_ctx *ctx, const void *x_dev, int rows, const void *w_dev,
                               const void *scales_dev, const void *biases_dev, int scale_dtype,
                               int group_size, int bits, int64_t n, int64_t k, int route,
                               void *y_dev, void *stream);
/* MLX dequantized(..., mode: .affine) as the reference's embedding path uses it
 * (Hadamard.swift:378-381): w = float(code) * scale + bias, fp32 out [n, k]. */
ishi_status ishi_affine_dequantize(ishi_ctx *ctx, const void *w_dev, const void *scales_dev,
                                   const void *biases_dev, int scale_dtype, int group_size,
                                   int bits, int64_t n, int64_t k, float *out_dev, void *stream);
/* hadamardRotate(x, block:, signs:) forward form (Hadamard.swift:8-23). */
ishi_status ishi_hadamard_rotate(ishi_ctx *ctx, const void *x_dev, int64_t rows, int64_t width,
                                 int block, const float *signs_dev, void *y_dev, void *stream);
/* VerifyMatmul.minimumRows(bytes:) exactly as the reference tabulates it for Apple M1
 * (VerifyMatmul.swift:19-26); kept so a host can reproduce the reference's routing. */
int ishi_reference_minimum_rows(int64_t bytes);
/* GGMLType.blockSize / typeSize (GGUFFile.swift:44-80); 0 for a type this library lacks. */
int ishi_ggml_block_size(int ggml_type);
int ishi_ggml_type_size(int ggml_type);

/* ---- for callers that cannot allocate --------------------------------------------------------- */

/* Has no counterpart in the reference. x [rows, k] against raw Q4_K blocks [n][k/256][144], like
 * ishi_ggml_matmul_few, for a host that has no way to obtain device memory of its own beyond the
 * buffers it is handed: a plugin running inside another runtime that reserved the whole GPU up
 * front and hands out fixed input/output buffers, or a serving loop whose rules forbid allocation
 * after start-up. Such a caller cannot create a context or a projection, since both allocate,
 * so this entry point takes none: it works on the current device and everything the kernel needs
 * besides x, the blocks and y (the re-tiled copy of the weight, the partial sums of panels shared
 * between CTAs, their arrival counters, the error word) lives in one 16 MiB array that is part
 * of the library image on every GPU that loads it. It calls no cudaMalloc, cudaFree or any other
 * allocating routine.
 *
 * Limits: rows 1...16, k a multiple of 256, and the weight at most 12 MiB of blocks
 * (n * k/256 * 144 bytes with n rounded up to a multiple of 128); anything larger returns
 * ISHI_E_TOO_LARGE and launches nothing. (The array's other parts, arrival counters for 131072
 * output rows and 3.9 MiB of partial sums, cannot fill up before the weight part does.) A device
 * that is not sm_100 returns ISHI_E_UNSUPPORTED.
 *
 * The first call on a device looks up the array's device address and sets the kernel's
 * shared-memory limit. Every call ends by synchronising the stream and reading the error word
 * back, so it returns when y is complete and it can never be part of a stream capture. All calls
 * on a device share the one array and it keeps whatever the last call left in it: the counters
 * and the error word are cleared at the start of every call, the rest is overwritten before it is
 * read. Two calls that overlap on the same GPU (two host threads, two streams) race on it:
 * serialise them. */
ishi_status ishi_q4k_matmul_few_static(const void *x_dev, int rows, const void *blocks_dev,
                                       int64_t blocks_bytes, int64_t n, int64_t k, void *y_dev,
                                       void *stream);

/* ---- N-sharded projections: output exchange over NVLink ---------------------------------------
 *
 * The reference runs on one GPU; these have no counterpart in it. Each rank (one process per GPU)
 * holds the rows [r*N/G, (r+1)*N/G) of every projection (desc.n = rows of the shard). Instead of
 * a collective after the product, the product kernel stores its rows into every rank's copy of
 * the output through peer mappings, and the ranks tell each other with arrival words: no extra
 * kernel, nothing on the host, the whole step can be one CUDA graph.
 *
 * An exchange owns, on every rank, one buffer of out_bytes for outputs and a few arrival words.
 * Outputs are fp16 arrays [rows of all shards][8]: row n holds the (up to 8) drafted rows'
 * values of output n, the transposed form of ishi_projection_apply; a call with 9...16 drafted
 * rows uses [rows of all shards][16] instead (two launches). All ranks must issue the same
 * sequence of ishi_exchange_apply calls. Waits on the device are bounded (about a second) and
 * raise the context's error word (ishi_ctx_poll) instead of hanging. */
typedef struct ishi_exchange ishi_exchange;
enum { ISHI_EXCHANGE_HANDLE_BYTES = 128 };
/* Allocates this rank's buffer (cudaMalloc) and arrival words. */
ishi_status ishi_exchange_create(ishi_ctx *ctx, int rank, int world, int64_t out_bytes,
                                 ishi_exchange **out);
/* Writes ISHI_EXCHANGE_HANDLE_BYTES bytes the other ranks need to map this rank's buffers (CUDA
 * IPC handles); the host passes them around by any means it has. */
ishi_status ishi_exchange_export(ishi_exchange *ex, void *handle_out);
/* handles: world x ISHI_EXCHANGE_HANDLE_BYTES, rank by rank (this rank's own entry is ignored). */
ishi_status ishi_exchange_connect(ishi_exchange *ex, const void *handles);
/* This rank's output buffer (device pointer). */
void *ishi_exchange_buffer(ishi_exchange *ex);
/* x [rows, k] (rows 1...16) against this rank's shard; the rows land at
 * buffer + out_offset_bytes, rows [row_offset, row_offset + n) of the [.][8] array ([.][16] when
 * rows > 8), on every rank.
 * wait_previous != 0: the kernel first waits until every rank's previous ishi_exchange_apply has
 * landed here (use it when x was produced from exchanged outputs). */
ishi_status ishi_exchange_apply(ishi_exchange *ex, ishi_projection *p, const void *x_dev, int rows,
                                int64_t out_offset_bytes, int64_t row_offset, int wait_previous,
                                void *stream);
/* Enqueues a wait for every rank's latest ishi_exchange_apply to have landed in this rank's buffer. */
ishi_status ishi_exchange_wait(ishi_exchange *ex, void *stream);
/* Test hook: makes this rank expect `launches_ahead` more launches than were issued, so that the
 * next ishi_exchange_wait waits for arrival words nobody will write. The wait gives up after its
 * bound (about a second), raises the context's error word and returns: this is how the
 * failure path of the bounded waits is exercised without hanging or faulting a GPU. */
ishi_status ishi_exchange_debug_expect(ishi_exchange *ex, unsigned launches_ahead);
/* Teardown in two steps, because the other ranks hold mappings of this rank's buffer and may
 * still be storing into it: every rank calls ishi_exchange_disconnect (waits for its own launches,
 * closes its mappings of the peers' buffers; apply is refused afterwards), the HOST then barriers
 * across the ranks by whatever channel it has, and only then every rank calls
 * ishi_exchange_destroy, which frees the buffer. destroy alone disconnects first, which is enough
 * for a single rank. */
ishi_status ishi_exchange_disconnect(ishi_exchange *ex);
void ishi_exchange_destroy(ishi_exchange *ex);

/* ---- GGUF container ----------------------------------------------------------------------------
 *
 * GGUFFile (Sources/IshizukiKit/Config/GGUFFile.swift:179-397): header, metadata and tensor table
 * of a .gguf file, the tensor data left on disk until a tensor is asked for. Host only (no GPU
 * needed) except ishi_gguf_upload_tensor. The reference's refusals are kept: versions other than
 * 2 and 3, implausible counts and lengths, ranks outside 1...4, unknown tensor types, shapes that
 * are not whole blocks, an alignment that is not a power of two. */
typedef struct ishi_gguf ishi_gguf;
typedef struct ishi_gguf_tensor_info {
  const char *name;   /* valid while the file is open */
  int32_t rank;       /* 1...4 */
  int64_t shape[4];   /* row-major (the file stores the fastest-varying dimension first): a
                         [5120, 248320] table in the file reads as 248320 rows of 5120 here */
  int32_t ggml_type;
  int64_t offset;     /* relative to ishi_gguf_data_offset */
  int64_t byte_count;
} ishi_gguf_tensor_info;
/* error_out (may be NULL) receives the reason when the file is refused. */
ishi_status ishi_gguf_open(const char *path, ishi_gguf **out, char *error_out, size_t error_len);
void ishi_gguf_close(ishi_gguf *g);
const char *ishi_gguf_last_error(const ishi_gguf *g);
uint32_t ishi_gguf_version(const ishi_gguf *g);
int64_t ishi_gguf_data_offset(const ishi_gguf *g);
int64_t ishi_gguf_alignment(const ishi_gguf *g);
int64_t ishi_gguf_tensor_count(const ishi_gguf *g);
int64_t ishi_gguf_find_tensor(const ishi_gguf *g, const char *name); /* index, or -1 */
ishi_status ishi_gguf_tensor(const ishi_gguf *g, int64_t index, ishi_gguf_tensor_info *out);
/* GGMLType.blockSize / typeSize / name for every type of the file format (GGUFFile.swift:44-113,
 * pinned by Tests/IshizukiKitTests/GGUFTests.swift:17-35); 0 / NULL for an unknown id. */
int ishi_gguf_type_block_size(int ggml_type);
int ishi_gguf_type_size(int ggml_type);
const char *ishi_gguf_type_name(int ggml_type);
/* Metadata (GGUFValue): kind is 0 when the key is absent, else 1 uint, 2 int, 3 float, 4 bool,
 * 5 string, 6 array. The int getter converts like GGUFValue.intValue. */
int64_t ishi_gguf_metadata_count(const ishi_gguf *g);
const char *ishi_gguf_metadata_key(const ishi_gguf *g, int64_t index);
int ishi_gguf_metadata_kind(const ishi_gguf *g, const char *key);
ishi_status ishi_gguf_metadata_int(const ishi_gguf *g, const char *key, int64_t *out);
ishi_status ishi_gguf_metadata_float(const ishi_gguf *g, const char *key, double *out);
const char *ishi_gguf_metadata_string(const ishi_gguf *g, const char *key);
int64_t ishi_gguf_metadata_array_length(const ishi_gguf *g, const char *key); /* -1: not an array */
ishi_status ishi_gguf_metadata_array_int(const ishi_gguf *g, const char *key, int64_t index, int64_t *out);
const char *ishi_gguf_metadata_array_string(const ishi_gguf *g, const char *key, int64_t index);
/* GGUFFile.data(for:): the bytes of one tensor into host memory. */
ishi_status ishi_gguf_read_tensor(ishi_gguf *g, int64_t index, void *dst_host, int64_t dst_bytes);
/* The same into device memory (the blocks a projection is created from, GGUFWeights.load,
 * Sources/IshizukiKit/Core/GGUFWeights.swift:47-85), through page-locked staging; returns when the
 * last copy has been issued and its staging buffer is free again. */
ishi_status ishi_gguf_upload_tensor(ishi_gguf *g, int64_t index, void *dst_dev, int64_t dst_bytes, void *stream);

/* ---- N-sharded projections: one NCCL all-gather per projection --------------------------------
 *
 * The plain way to assemble an N-sharded projection (no counterpart in the single-GPU reference):
 * every rank multiplies its rows and one ncclAllGather of the fp16 rows gives every rank the whole
 * output. A group owns one NCCL communicator in non-blocking mode; NCCL is loaded at run time
 * (libnccl.so.2), a host without it gets ISHI_E_UNSUPPORTED. Nothing here blocks for ever: a rank
 * that never arrives ends in ISHI_E_TIMEOUT after timeout_ms and the communicator is aborted. */
typedef struct ishi_group ishi_group;
enum { ISHI_GROUP_ID_BYTES = 128 };
/* Rank 0 calls this (ncclGetUniqueId) and hands the bytes to every rank by any means it has. */
ishi_status ishi_group_unique_id(void *id_out);
/* All ranks call this with the same id, on the GPU that is current for the calling thread. A group
 * is returned even on failure when its message is worth reading (destroy it as usual). */
ishi_status ishi_group_create(const void *id, int rank, int world, int timeout_ms, ishi_group **out);
const char *ishi_group_last_error(const ishi_group *g);
/* x [rows, k] against this rank's shard p (n_local rows, the same on every rank): y_all_dev is
 * fp16 [world * n_local][rows], rank r's rows at [r * n_local, (r + 1) * n_local), the transposed
 * form of ishi_projection_apply; the product writes this rank's slab in place and the all-gather
 * fills the rest, both on the stream. rows in 1...16. Eager streams only: on a stream that is being
 * captured into a CUDA graph the call returns ISHI_E_UNSUPPORTED (ishi_exchange_apply can be captured). */
ishi_status ishi_projection_apply_sharded(ishi_group *g, ishi_projection *p, const void *x_dev, int rows,
                                          void *y_all_dev, void *stream);
void ishi_group_destroy(ishi_group *g);
/* Test hook: replaces the NCCL entry points the library uses by the table given (seven function
 * pointers in the order ncclGetUniqueId, ncclCommInitRankConfig, ncclCommGetAsyncError,
 * ncclAllGather, ncclCommAbort, ncclCommDestroy, ncclGetErrorString), or restores the real ones
 * with NULL. Lets the error and time-out paths be exercised on a machine without GPUs. */
ishi_status ishi_group_debug_set_api(const void *table);

/* ---- layer stages around the projections --------------------------------------------------- */

/* The RMS norm ahead of q/k/v and of gate/up (MLXFast.rmsNorm in DecoderLayer.callAsFunction,
 * Sources/IshizukiKit/Text/TextModel.swift:151-161): y [rows, width] fp16 =
 * x * rsqrt(mean(x^2) + eps) * weight, fp32 inside. x fp32 (the reference's residual stream) or
 * fp16; weight [width] fp16, bf16 or fp32; width up to 8192. One launch that joins the stream's
 * chain of dependent launches (it starts while the launch before it drains, and the product after
 * it runs its own prologue meanwhile). silu(gate) * up, the other stage of the MLP, is part of
 * ishi_projection_create_gated. */
ishi_status ishi_rms_norm(ishi_ctx *ctx, const void *x, int x_dtype, int64_t rows, int64_t width, const void *weight,
                          int weight_dtype, float eps, void *y, void *stream);

/* ---- EXL3 trellis-coded projections: EXL3Tensor / EXL3Kernels ------------------------------ */

enum { ISHI_EXL3_3INST = 0, ISHI_EXL3_MCG = 1, ISHI_EXL3_MUL1 = 2 };

/* EXL3Tensor (Sources/IshizukiKit/Core/EXL3.swift:9-79). The weight is W [k, n] in 16 x 16 tiles
 * of 16 * bits int16 each; bits in {1, 1.5, 2, 2.5, 3, 3.5, 4, 5, 6, 7, 8}, the half rates only with
 * the MUL1 codebook; k and n whole numbers of 128 (EXL3.swift:28-49: ISHI_E_SHAPE /
 * ISHI_E_UNSUPPORTED otherwise). The scale vectors are fp16 (the unpacked "suh" / "svh" form). */
typedef struct ishi_exl3_desc {
  const int16_t *trellis_dev;     /* [k / 16][n / 16][words_per_tile] */
  int64_t k, n;
  int32_t words_per_tile;         /* 16 * bits */
  int32_t codebook;               /* ISHI_EXL3_* */
  const void *input_scales_dev;   /* fp16 [k]; may be NULL for the kernel-level calls that do not rotate */
  const void *output_scales_dev;  /* fp16 [n] */
} ishi_exl3_desc;

/* EXL3Kernels.dequantize (EXL3.swift:124-141, 275-292): W [k, n] as fp16 or fp32 (ISHI_DT_F16 /
 * ISHI_DT_F32), bit-exact against the exllamav3 reconstruction in the reference's fixture. */
ishi_status ishi_exl3_dequantize(ishi_ctx *ctx, const ishi_exl3_desc *t, int out_dtype, void *w_out, void *stream);
/* EXL3Kernels.rotate (EXL3.swift:108-122, 219-262): block Hadamard of 128 along each row, times
 * 1 / sqrt(128), with the fp16 scale vector applied first (before != 0) or last; fp32 inside.
 * x and y: [rows, width], fp16 or fp32 each. */
ishi_status ishi_exl3_rotate(ishi_ctx *ctx, const void *x, int x_dtype, int64_t rows, int64_t width,
                             const void *scales_dev, int before, void *y, int y_dtype, void *stream);
/* EXL3Kernels.matvec (EXL3.swift:143-163, 294-343): y [rows, n] fp32 = x [rows, k] fp16 . W for
 * 1...8 rows, the tiles decoded straight into tensor-core operands (a tile's weight order is the
 * A fragment of mma.sync m16n8k16 with n on the M side); no rotation. */
ishi_status ishi_exl3_matvec(ishi_ctx *ctx, const ishi_exl3_desc *t, const void *x, int rows, float *y, void *stream);
/* EXL3Kernels.apply (EXL3.swift:83-106): rotate x with the input scales (to fp16), multiply, rotate
 * the fp32 product with the output scales; y [rows, n] fp16, 1...16 rows (9...16 as two products,
 * as the reference does; its dense route above 16 rows is not part of this library: ISHI_E_SHAPE).
 * Uses scratch of the context, grown on demand by the first call of a larger shape (which then
 * allocates and must not be captured into a graph). */
ishi_status ishi_exl3_apply(ishi_ctx *ctx, const ishi_exl3_desc *t, const void *x, int rows, void *y, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ISHIZUKI_CUDA_H */
