// Instantiates the warp-level kernel for one fragment decoder and wraps its launches in a FragOps
// table (see ishi_kernels.h). Included by the frag_*.cu translation units only.
#pragma once
#include <cstring>

#include "ishi_kernels.h"

namespace ishi {

template <class Fmt>
struct FragOpsOf {
  static cudaError_t configure(int max_smem) {
    const auto attr = cudaFuncAttributeMaxDynamicSharedMemorySize;
    cudaError_t e = cudaFuncSetAttribute(frag_kernel<Fmt, 0, kFragFewWarps>, attr, max_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(frag_kernel<Fmt, 0, kFragMaxWarps>, attr, max_smem);
    if constexpr (Fmt::kRowMode) {
      if (e == cudaSuccess) e = cudaFuncSetAttribute(frag_kernel<Fmt, 1, kFragFewWarps>, attr, max_smem);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(frag_kernel<Fmt, 1, kFragMaxWarps>, attr, max_smem);
    }
    return e;
  }

  static void fill(cudaLaunchConfig_t *cfg, cudaLaunchAttribute *at, int clusters, int split, int warps, size_t smem) {
    memset(cfg, 0, sizeof(*cfg));
    cfg->gridDim = dim3((unsigned)(clusters * split), 1, 1);
    cfg->blockDim = dim3((unsigned)(warps * 32), 1, 1);
    cfg->dynamicSmemBytes = smem;
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)split;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg->attrs = at;
    cfg->numAttrs = 1;
  }

  static int max_clusters(int split, int warps, size_t smem, int sm_count) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute at[2];
    fill(&cfg, at, sm_count, split, warps, smem);
    int n = 0;
    const cudaError_t e = warps <= kFragFewWarps
                              ? cudaOccupancyMaxActiveClusters(&n, frag_kernel<Fmt, 0, kFragFewWarps>, &cfg)
                              : cudaOccupancyMaxActiveClusters(&n, frag_kernel<Fmt, 0, kFragMaxWarps>, &cfg);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    return n;
  }

  static cudaError_t launch(const FragLaunch &l, const FragArgs &args) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute at[2];
    fill(&cfg, at, l.clusters, l.split, l.warps, l.smem);
    cfg.stream = l.stream;
    // Programmatic dependent launch: the kernel may start while the one before it on the stream
    // drains. It prefetches weight tiles, which no earlier kernel writes, and waits for the earlier
    // kernels before it touches x or y.
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = l.early ? 2 : 1;
    // a format without a CUDA-core variant for one activation row runs that row through the MMA path
    const bool few = l.warps <= kFragFewWarps;
    if constexpr (Fmt::kRowMode) {
      if (l.mode == 1)
        return few ? cudaLaunchKernelEx(&cfg, frag_kernel<Fmt, 1, kFragFewWarps>, args)
                   : cudaLaunchKernelEx(&cfg, frag_kernel<Fmt, 1, kFragMaxWarps>, args);
    }
    return few ? cudaLaunchKernelEx(&cfg, frag_kernel<Fmt, 0, kFragFewWarps>, args)
               : cudaLaunchKernelEx(&cfg, frag_kernel<Fmt, 0, kFragMaxWarps>, args);
  }

  static cudaError_t prepare(const FragSrc &src, int units, uint8_t *dst, int grid, cudaStream_t stream) {
    prepare_frag_kernel<Fmt><<<grid, 256, 0, stream>>>(src, units, Fmt::kTileBytes, dst);
    return cudaGetLastError();
  }

  static constexpr FragOps ops() {
    return FragOps{Fmt::kTileBytes, Fmt::kXBytes, Fmt::kExtraBytes, &configure, &max_clusters, &launch, &prepare};
  }
};

}  // namespace ishi
