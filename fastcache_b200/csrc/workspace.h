// Scratch memory of the kernels that need some (split-K partial sums and arrival counters of the GEMMs, the
// grid barrier of the fused GEMM epilogues, split-KV partials of decode attention).
//
// One set per (device, stream): two streams that run decode-size GEMMs or decode attention at the same time
// (a compression stream beside the main stream, the side streams of PipelineAsyncCompressor) must not share
// partial sums or counters.  The status word is per device.  Sets are created on first use of a stream; the
// first use must therefore not happen inside a CUDA-graph capture (the engine warms every captured shape up
// on the capturing stream first).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fc {

struct StreamWorkspace {
  float* gemm_scratch = nullptr;     // gemm_scratch_bytes()
  int* gemm_counters = nullptr;      // gemm_counter_bytes(), zero between launches
  uint32_t* grid_sync = nullptr;     // [2] arrival count and generation of the in-kernel grid barrier
  float* attn_o = nullptr;           // ATTN_WS_FLOATS
  float* attn_lse = nullptr;         // ATTN_LSE_FLOATS
  int* attn_counters = nullptr;      // ATTN_COUNTERS arrival counters of the split-KV merge, zero between launches
  uint32_t* status = nullptr;        // the device's status word
};

constexpr long long ATTN_WS_FLOATS = 4ll << 20;   // 16 MiB of split-KV partial outputs
constexpr long long ATTN_LSE_FLOATS = 1ll << 18;
constexpr long long ATTN_COUNTERS = 1ll << 16;    // (requests x KV heads) of one decode batch

// Implemented in bindings.cpp (the memory is owned by torch tensors).
const StreamWorkspace& stream_workspace(int device, cudaStream_t stream);
// SM count of the green context a stream belongs to (0: the whole device).
int stream_sm_limit(cudaStream_t stream);
// true after set_fused_epilogues(true), or initially when the environment variable FC_FUSED_EPILOGUE is 1: the decode-size row-parallel GEMMs then run their
// (all-reduce +) add + RMSNorm inside the GEMM kernel instead of as a second kernel (see bindings.cpp for why
// the default is the pair).
bool fused_epilogues_enabled();
void set_fused_epilogues(bool on);

}  // namespace fc
