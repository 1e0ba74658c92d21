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
  // > 0: "push" form of the one-shot all-reduce.  Every staging buffer then holds `world` slots of `slot_rows`
  // token rows, slot s for the rows that rank s sends: a rank stores its finished row into slot `rank` of EVERY
  // peer before the flag exchange and afterwards sums the slots of its own buffer, instead of fetching the
  // peers' rows with loads over NVLink after the exchange.
  int slot_rows;
  // > 0: "two-shot" form through NVSwitch multicast.  Rows [reduced_row0, ...) of every staging buffer receive the
  // reduced rows: the owner of a token row (row % world) sums all ranks' copies of it inside the switch
  // (multimem.ld_reduce) and publishes the sum to every rank with one multimem.st; a second flag exchange tells
  // the others that it is there.  Each rank then receives one row's worth of bytes per row instead of world - 1.
  int reduced_row0;
};

// Candidate tables of the sampler over vocabulary shards: per rank [2][COMM_MAX_SLOTS][COMM_MAX_WORLD] 8-byte
// cells (value bits << 32 | global token index) in symmetric memory.
struct SamplePeers {
  uint64_t* cells[COMM_MAX_WORLD];
};
constexpr size_t SAMPLE_CELLS_PER_RANK = size_t(2) * COMM_MAX_SLOTS * COMM_MAX_WORLD;

// logits [B, V] are this rank's shard (vocabulary entries vocab_offset ... vocab_offset + V - 1, entries >= v_limit
// are padding); out int64 [B + 1]: the tokens, identical on every rank, then the device status code.
void launch_sample_exchange(const CommPeers& peers, const SamplePeers& cand, const void* logits, const void* temps,
                            void* out, int B, int V, long long ld, uint32_t seed, int vocab_offset, int v_limit,
                            uint32_t* epochs, uint32_t* status, cudaStream_t stream);

void launch_allreduce_add_rmsnorm(const CommPeers& peers, int buf, const void* mc_in, void* residual,
                                  const void* weight, void* out, int T, int H, float eps, uint32_t* epochs,
                                  uint32_t* status, bool use_multimem, cudaStream_t stream,
                                  const float* partial = nullptr, int splits = 0, long long split_stride = 0,
                                  const void* bias = nullptr);
// `partial` != nullptr: this rank's contribution is still fp32 split-K partial sums [splits, T, H] (plus an optional
// bias); each CTA finishes its rows into the staging buffer before it joins the exchange.

}  // namespace fc

namespace fc {

// Symmetric buffers of the prefill-size fused GEMM + collective kernels (gemm_tp.cu).
struct TpBuffers {
  int world = 1;
  int rank = 0;
  __nv_bfloat16* stage[COMM_MAX_WORLD] = {};        // per rank: [world][chunk_rows_max][hidden] partial sums by source
  __nv_bfloat16* xg[COMM_MAX_WORLD] = {};           // per rank: gathered normalised activations [max_tokens][hidden]
  uint32_t* rs_flags[COMM_MAX_WORLD] = {};          // per rank: [world] "source s delivered its partials"
  uint32_t* gathered_flags[COMM_MAX_WORLD] = {};    // per rank: [world] "owner o's rows have landed here"
  int* owner_done = nullptr;                        // local [world + 1] counters, zero between calls
  // pipelined reduce-scatter: per 128-row group of a chunk
  uint32_t* group_flags[COMM_MAX_WORLD] = {};       // per rank: [max_groups][COMM_MAX_WORLD] "source s delivered group g"
  int* group_done = nullptr;                        // local [world][max_groups] counters, zero between calls
  int max_groups = 0;
  // NVSwitch multicast addresses of the staging / gathered buffers (nullptr: none)
  const __nv_bfloat16* stage_mc = nullptr;
  __nv_bfloat16* xg_mc = nullptr;
};

// The row-parallel GEMM reduces each 128-row group as soon as all ranks have delivered it (only when
// FC_TP_PIPELINE=1 or after set_tp_pipeline(true)); otherwise one reduction phase after the GEMM.
bool tp_pipeline_enabled();
void set_tp_pipeline(bool on);
// The pipelined form sums through the switch (multimem.ld_reduce / multimem.st) when the buffers have multicast
// addresses (on unless FC_TP_NVLS=0).
bool tp_nvls_enabled();
void set_tp_nvls(bool on);

// Row-parallel GEMM + reduce-scatter + residual add + RMSNorm + send half of the all-gather.
// x [M, K] and w [N, K] are this rank's shards; `residual` holds the rows owned by this rank
// ([min(M - rank * chunk_rows, chunk_rows), N]) and is updated in place.  The normalised rows of all
// ranks arrive in xg (rows [0, M)) on every rank; consume them with gemm_after_gather or after
// wait_gathered.
void gemm_rs_add_norm(const void* x, const void* w, int M, int N, int K, long long ldx, long long ldw,
                      const TpBuffers& b, void* residual, const void* norm_w, float eps, int chunk_rows,
                      uint32_t epoch, uint32_t* status, int sm_limit, cudaStream_t stream);

// Column-parallel GEMM over the gathered activations: c [M, N] = xg[:M] @ w[N, K]^T.  Tiles of a
// chunk are loaded only after its owner's "gathered" flag for `epoch` has been observed.
void gemm_after_gather(const void* xg_local, const void* w, void* c, int M, int N, int K, long long ldw,
                       long long ldc, const TpBuffers& b, int chunk_rows, uint32_t epoch, uint32_t* status,
                       int sm_limit, cudaStream_t stream, bool swiglu = false);
// swiglu: w = [gate; up] stacked on dim 0; c [M, N / 2] = silu(xg gate^T) * (xg up^T), applied in the epilogue.

// Blocks the stream (one tiny kernel, bounded wait) until every owner's rows of `epoch` have landed.
void wait_gathered(const TpBuffers& b, uint32_t epoch, uint32_t* status, cudaStream_t stream);

}  // namespace fc
