// Instantiates the tcgen05 kernel for one row decoder and wraps its launches in a RowOps table
// (see ishi_kernels.h). Included by the row_*.cu translation units only.
#pragma once
#include "ishi_kernels.h"

namespace ishi {

template <class Fmt>
struct RowOpsOf {
  static cudaError_t configure(int max_smem) {
    cudaError_t e = cudaFuncSetAttribute(rowstream_kernel<Fmt, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(rowstream_kernel<Fmt, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(rowstream_kernel<Fmt, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(rowstream_kernel<Fmt, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    return e;
  }
  // the instance that keeps as many accumulator columns as there are activation rows
  static cudaError_t launch(int rows, int grid, size_t smem, const RowArgs &args, cudaStream_t st) {
    if (rows <= 1) rowstream_kernel<Fmt, 1><<<grid, kRowThreads, smem, st>>>(args);
    else if (rows <= 2) rowstream_kernel<Fmt, 2><<<grid, kRowThreads, smem, st>>>(args);
    else if (rows <= 4) rowstream_kernel<Fmt, 4><<<grid, kRowThreads, smem, st>>>(args);
    else rowstream_kernel<Fmt, 8><<<grid, kRowThreads, smem, st>>>(args);
    return cudaGetLastError();
  }
  static constexpr RowOps ops() { return RowOps{Fmt::kTableBytes, &configure, &launch}; }
};

}  // namespace ishi
