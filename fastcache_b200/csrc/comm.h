// Host interface of the fused tensor-parallel communication kernels (comm.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fc {

constexpr int COMM_MAX_WORLD = 8;
constexpr int COMM_MAX_SLOTS = 512;   // CTAs that take part in a flag exchange (all co-resident)

// Peer pointers into symmetric memory; passed to kernels by value.
struct CommPeers {
  int world;
  int rank;
  __nv_bfloat16* data[2][COMM_MAX_WORLD];   // two staging buffers per rank, used in alternation
  uint32_t* flags[COMM_MAX_WORLD];          // [COMM_MAX_SLOTS][COMM_MAX_WORLD] words per rank
};

void launch_allreduce_add_rmsnorm(const CommPeers& peers, int buf, const void* mc_in, void* residual,
                                  const void* weight, void* out, int T, int H, float eps, uint32_t* epochs,
                                  uint32_t* status, bool use_multimem, cudaStream_t stream);

}  // namespace fc
