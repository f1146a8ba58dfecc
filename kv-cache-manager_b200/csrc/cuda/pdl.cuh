// Programmatic dependent launch: a kernel launched this way may start while its predecessor in
// the stream is still running.  Before it touches anything the predecessor wrote it calls
// pdl_wait(), which returns once the predecessor has completed and its writes are visible; what
// it does before that (address arithmetic, loads of constants such as weights) overlaps with the
// predecessor's tail.  Every kernel of the decode path calls pdl_launch_dependents() first, which
// lets the *next* kernel be scheduled as soon as there is room.  A kernel that is launched the
// ordinary way simply waits for full completion, so mixing both kinds is always correct.
// Rule: a kernel launched through pdl_launch writes global memory only after pdl_wait().
#pragma once
#include <cuda_runtime.h>

namespace kvcm {

__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
}

template <typename Kernel, typename... Args>
int pdl_launch(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, args...));
}

// The same with the grid cut into thread-block clusters of `cluster_x` blocks along x (which must
// divide grid.x; at most 8).
template <typename Kernel, typename... Args>
int pdl_launch_cluster(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_x,
                       Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster_x;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, args...));
}

}  // namespace kvcm
