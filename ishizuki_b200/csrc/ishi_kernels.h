// What the C-ABI layer knows of the product kernels: one table of plain functions per weight
// format, defined in that format's own translation unit (frag_*.cu for the warp-level kernel,
// row_*.cu for the tcgen05 kernel) so that the formats compile side by side.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "ishi_fragstream.cuh"
#include "ishi_rowstream.cuh"

namespace ishi {

struct FragLaunch {
  int clusters, split, warps;  // grid = clusters * split CTAs of warps * 32 threads
  size_t smem;
  int mode;    // 0: tensor cores, rows 1..8; 1: CUDA cores, one row
  bool early;  // programmatic dependent launch
  cudaStream_t stream;
};

struct FragOps {
  int tile_bytes, x_bytes, x_extra;  // bytes per tile; activation staging per unit of the column range, and per CTA
  // raises the dynamic shared memory limit of every variant (once per device)
  cudaError_t (*configure)(int max_smem);
  // how many clusters of `split` CTAs the device keeps resident, 0 if the launch is impossible
  int (*max_clusters)(int split, int warps, size_t smem, int sm_count);
  cudaError_t (*launch)(const FragLaunch &cfg, const FragArgs &args);
  // the one-time re-tiling into fragment order
  cudaError_t (*prepare)(const FragSrc &src, int units, uint8_t *dst, int grid, cudaStream_t stream);
};

struct RowOps {
  int table_bytes;
  cudaError_t (*configure)(int max_smem);
  cudaError_t (*launch)(int rows, int grid, size_t smem, const RowArgs &args, cudaStream_t stream);
};

// ---- every GGML block format through the shared decoders (ggml_generic.cu) -----------------------
// out_dtype: 0 fp16, 1 bf16, 2 fp32
int ggml_type_size(int type);  // bytes of a 256-weight block, 0 for a type without a decoder
cudaError_t launch_ggml_dequantize(int type, const uint8_t *blocks, long long n_blocks, void *out, int out_dtype, int sm_count,
                                   cudaStream_t st);
cudaError_t launch_ggml_gather(int type, const int *ids, long long count, const uint8_t *blocks, long long table_rows,
                               long long k, void *out, int out_dtype, int sm_count, cudaStream_t st);
cudaError_t launch_ggml_rowdot(int type, const uint8_t *blocks, long long n, long long k, const __half *x, int rows, __half *y,
                               long long ldy, int transposed, int sm_count, cudaStream_t st);
size_t argmax_scratch_bytes();  // zeroed once; launch_argmax_rows leaves it zeroed
cudaError_t launch_argmax_rows(const __half *y, int rows, long long n, long long ldy, int *out, void *scratch, cudaStream_t st);

// ---- layer stages around the projections (ishi_stages.cu) -----------------------------------------
long long rms_norm_max_width();
cudaError_t launch_rms_norm(const void *x, int x_dtype, const void *w, int w_dtype, long long rows, long long width, float eps,
                            __half *y, cudaStream_t st);

// ---- EXL3 trellis-coded weights (ishi_exl3.cu) ---------------------------------------------------
// words16: int16 words per 16 x 16 tile (16 * bits); codebook: 0 3INST, 1 MCG, 2 MUL1; dtypes: 0 fp16, 2 fp32
bool exl3_rate_supported(int words16, int codebook);
cudaError_t launch_exl3_dequantize(const int16_t *trellis, int tiles_k, int tiles_n, int words16, int codebook, void *out,
                                   int out_dtype, int sm_count, cudaStream_t st);
cudaError_t launch_exl3_matvec(const int16_t *trellis, int tiles_k, int tiles_n, int words16, int codebook, const __half *x,
                               int rows, float *y, int sm_count, cudaStream_t st);
cudaError_t launch_exl3_rotate(const void *x, int x_dtype, long long rows, long long width, const __half *scales, int before,
                               void *y, int y_dtype, int sm_count, cudaStream_t st);

}  // namespace ishi
