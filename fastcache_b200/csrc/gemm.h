// Host interface of the tcgen05 GEMM (gemm.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fc {

enum Act : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_GELU_TANH = 3, ACT_QUICK_GELU = 4, ACT_SILU = 5,
                 ACT_SWIGLU = 6 };   // w = [gate; up]: out[M, N/2] = silu(x gate^T) * (x up^T), M > 256 only

// Split-K needs scratch for fp32 partial tiles and one arrival counter per output
// tile (zero before the first launch; the kernel leaves them zero).
constexpr int GEMM_SCRATCH_TILES = 512;     // (tile, split) partials that fit the scratch
constexpr int GEMM_MAX_TILES_SPLIT = 4096;  // counters

struct GemmWorkspace {
  float* scratch = nullptr;
  int* counters = nullptr;
  uint32_t* status = nullptr;
  uint32_t* grid_sync = nullptr;   // [2] words of the in-kernel grid barrier (zero before the first launch)
};

// Epilogues fused into the decode-size GEMM (gemm_skinny.cu).
enum SkinnyEpilogue : int { EPI_NONE = 0, EPI_ADD_NORM = 1, EPI_AR_ADD_NORM = 2 };

struct CommPeers;
struct SkinnyFused {
  int epi = EPI_NONE;
  void* residual = nullptr;        // [M, N] bf16, updated in place
  const void* norm_w = nullptr;    // [N] bf16
  void* y = nullptr;               // [M, N] bf16: RMSNorm(residual) * norm_w
  float eps = 1e-6f;
  // EPI_AR_ADD_NORM: sum over the tensor-parallel ranks between the GEMM and the residual add
  const CommPeers* peers = nullptr;
  int buf = 0;                     // staging buffer of this call (the two are used in alternation)
  const void* mc_in = nullptr;     // multicast address of that buffer: multimem.ld_reduce instead of peer loads
  uint32_t* epochs = nullptr;
};

size_t gemm_scratch_bytes();
size_t gemm_counter_bytes();
int gemm_num_sms();

CUtensorMap make_tmap_bf16_2d(const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                              uint32_t box_cols);

// c[M, N] = act(x[M, K] @ w[N, K]^T + bias[N]); bf16 in/out, fp32 accumulate.
// ldx / ldw / ldc are row pitches in elements.  sm_limit > 0 caps the persistent grid
// (used when the launching stream belongs to a green context with fewer SMs).
void gemm_bf16(const void* x, const void* w, void* c, const void* bias, int M, int N, int K, long long ldx,
               long long ldw, long long ldc, int act, const GemmWorkspace& ws, int sm_limit, cudaStream_t stream);

// Decode-size batches (M <= 256).  Returns the number of K splits used; when that is > 1 and
// `finalize` is false, ws.scratch holds fp32 partial sums [splits, M, N] for the caller to reduce.
// `fused` != nullptr: the epilogue named there runs inside the kernel (`c` and `act` are unused).  Returns 0 without
// launching anything when the shape cannot take the fused form (more row tiles than SMs, hidden size above 8192 or
// not a multiple of 8): the caller then runs the unfused pair of kernels.
// `flags`: SK_SWIGLU: w = [gate; up] ([N, K], N = 2 x width) and c [M, N / 2] = silu(x gate^T) * (x up^T); needs
// width % 128 == 0 and the cluster form (returns 0 without launching when it cannot be taken).  SK_NO_CLUSTER: never
// reduce the K splits inside a thread-block cluster (done where the shape allows when cluster_splitk_enabled(): the
// result is then always finished bf16 in `c` and the return value is 1).
enum SkinnyFlags : int { SK_SWIGLU = 1, SK_NO_CLUSTER = 2 };
int gemm_skinny_bf16(const void* x, const void* w, void* c, const void* bias, int M, int N, int K, long long ldx,
                     long long ldw, long long ldc, int act, const GemmWorkspace& ws, int sm_limit,
                     int splits_request, bool finalize, cudaStream_t stream, const SkinnyFused* fused = nullptr,
                     int flags = 0);
// Split-K inside clusters on / off for the whole process (initially off unless FC_CLUSTER_SPLITK=1: it measured
// slower than partial sums through L2, see gemm_skinny.cu).
void set_cluster_splitk(bool on);
bool cluster_splitk_enabled();

// Persistent stream-K form for finished outputs (gemm_streamk.cu), M <= 128: c = act(x w^T + bias), or with `swiglu`
// w = [gate; up] ([N, K]) and c [M, N / 2] = silu(x gate^T) * (x up^T) (N % 256 == 0, no bias).  Returns false
// without launching when the shape cannot take it.  Mode (FC_STREAMK / set_streamk): 0 never, 1 (initial) where a row
// tile is cut into about three spans at most, 2 wherever the shape allows.
bool gemm_streamk_bf16(const void* x, const void* w, void* c, const void* bias, int M, int N, int K, long long ldx,
                       long long ldw, long long ldc, int act, bool swiglu, const GemmWorkspace& ws, int sm_limit,
                       cudaStream_t stream);
// Prefill sizes on CTA pairs (gemm_2cta.cu): one tcgen05.mma.cta_group::2 of 256 x 256 per pair of SMs.  M > 256,
// N >= 256, bias along N, any activation incl. ACT_SWIGLU.  Returns false without launching when it cannot run.
bool gemm_bf16_2cta(const void* x, const void* w, void* c, const void* bias, int M, int N, int K, long long ldx,
                    long long ldw, long long ldc, int act, int sm_limit, uint32_t* status, cudaStream_t stream);
int gemm_pairs_mode();            // FC_GEMM_PAIRS=1 / set_gemm_pairs(1): gemm_bf16 takes the pair form where it can
void set_gemm_pairs(int mode);
bool streamk_enabled();
void set_streamk(int mode);
int streamk_mode();

}  // namespace fc
