// Host-side kernel launch with the attributes this library uses: an optional cluster width and
// programmatic dependent launch (the kernel may be scheduled while its predecessor in the
// stream drains; every kernel launched through here calls grid_dependency_wait() before its
// first access to memory another kernel may write).
#pragma once
#include <cuda_runtime.h>

#include <utility>

namespace iflb200 {

// 0: plain stream order; 1 (default): dependent launch for kernels over at most
// kDependentLaunchMaxRows activation rows; 2: always.  Measured on B200: with a few hundred rows
// (kernels of 3-50 us) early scheduling of the next kernel shortens a layer stack by 5-15 %;
// with thousands of rows (kernels of 40-300 us) the same stack got 3-6 % slower.
extern int g_dependent_launch;
constexpr long long kDependentLaunchMaxRows = 2048;
inline bool dependent_launch_for(long long rows) {
  return g_dependent_launch == 2 || (g_dependent_launch == 1 && rows <= kDependentLaunchMaxRows);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                              int cluster_x, bool dependent, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (dependent) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace iflb200
