// Kernel launch with programmatic stream serialization: the kernel may be scheduled while the
// previous kernel of the stream drains, and orders itself with griddepcontrol.wait (ptx.cuh,
// `pdl_wait`).  Every kernel launched through here must call `pdl_wait()` before its first access to
// global memory.  Decode steps are chains of 5-50 microsecond kernels, where the launch gap and the
// prologue of each kernel are a visible share of the step; the launches are captured into the
// decode CUDA graphs as programmatic dependencies.
//
// The environment variable FC_PDL is a bit mask of the kernel families that use it (default: all);
// FC_PDL=0 launches everything the ordinary way.
#pragma once
#include <cuda_runtime.h>

#include <cstdlib>
#include <utility>

namespace fc {

enum PdlFamily : unsigned {
  PDL_SKINNY_GEMM = 1u << 0,
  PDL_FINALIZE = 1u << 1,
  PDL_PARTIALS = 1u << 2,
  PDL_NORM = 1u << 3,
  PDL_EMBEDDING = 1u << 4,
  PDL_ROPE = 1u << 5,
  PDL_SAMPLE = 1u << 6,
  PDL_DECODE_ATTN = 1u << 7,
  PDL_DECODE_MERGE = 1u << 8,
  PDL_ALLREDUCE = 1u << 9,
};

inline unsigned pdl_mask() {
  static const unsigned mask = [] {
    const char* e = std::getenv("FC_PDL");
    // Paged decode attention stays on ordinary launches by default: with it enabled, CUDA-graph decode
    // produced tokens that differed from eager decode (every other family, alone and together, matches)
    return e == nullptr ? (~0u & ~unsigned(PDL_DECODE_ATTN)) : unsigned(std::strtoul(e, nullptr, 0));
  }();
  return mask;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(unsigned family, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl_mask() & family) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

// The same with a thread-block cluster of (1, cluster_y, 1) CTAs (grid.y must be a multiple of cluster_y).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(unsigned family, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, unsigned cluster_y, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = cluster_y;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl_mask() & family) ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

}  // namespace fc
