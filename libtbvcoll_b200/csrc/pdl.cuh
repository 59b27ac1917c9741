// pdl.cuh — programmatic dependent launch (PDL) helpers.
//
// Every kernel of the decode step is launched with the "programmatic stream serialization"
// attribute: it may start while its predecessor in the stream is still running.  Each
// kernel (1) signals `launch_dependents` as early as it can, so that the next kernel's
// CTAs are resident, have set up their barriers / TMEM and — for GEMMs — are already
// streaming WEIGHT tiles (which no kernel ever writes) while this one finishes, and
// (2) executes `grid_dependency_wait` before it touches anything a predecessor produces.
// Because every kernel waits, completion is transitive: when kernel B has finished, every
// kernel before it has too.  Works inside CUDA graphs (captured as programmatic edges).
// TBV_PDL=0 turns the attribute off (plain stream order).
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

namespace pdl {

__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("TBV_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

// cudaLaunchKernelEx with the PDL attribute (and an optional cluster size along z).
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_z,
                          Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (cluster_z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = unsigned(cluster_z);
    n++;
  }
  if (enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    n++;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace pdl
