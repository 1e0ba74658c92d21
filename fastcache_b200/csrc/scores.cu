// KV scoring kernels that need no attention pass: ExpectedAttention (query statistics) and the
// position-only StreamingLLM scorer.
//
// Scores are fp32 [n_seq, L, Hkv, stride]; the selection kernel (evict.cu) only ranks them, so the
// ExpectedAttention score is kept in the log domain:
//     log score[c] = k_c . mu / sqrt(D) + k_c^T Sigma k_c / (2 D) + log ||v_c||
// which orders the keys exactly like exp(logit - max) * ||v|| of the kvpress statement.  mu and Sigma
// are the mean and the (unbiased) covariance of the observation-window queries of the G query heads
// that share the KV head.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

#include "kernels.h"
#include "ptx.cuh"

namespace fc {

using bf16 = __nv_bfloat16;

constexpr float SC_POS = 3.0e38f;

// ------------------------------------------------------------------ query statistics
// grid (Hkv, L, n_seq), 256 threads.  stats[unit] = mu[D] followed by Sigma[D][D].
template <int D>
__global__ void __launch_bounds__(256)
ea_stats_kernel(const bf16* __restrict__ qw, float* __restrict__ stats, int L, int Hkv, int Hq, int w) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int hk = blockIdx.x, layer = blockIdx.y, seq = blockIdx.z;
  const int G = Hq / Hkv, rows = G * w;
  float* s_q = reinterpret_cast<float*>(smem);               // [rows][D], centred
  float* s_mu = s_q + rows * D;                              // [D]
  const bf16* src = qw + (((long long)seq * L + layer) * w) * Hq * D;
  for (int i = threadIdx.x; i < rows * D; i += blockDim.x) {
    const int r = i / D, d = i % D;
    const int hg = r / w, wr = r % w;
    s_q[i] = __bfloat162float(src[((long long)wr * Hq + hk * G + hg) * D + d]);
  }
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < rows; ++r) acc += s_q[r * D + d];
    s_mu[d] = acc / float(rows);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < rows * D; i += blockDim.x) s_q[i] -= s_mu[i % D];
  __syncthreads();
  float* out = stats + (((long long)seq * L + layer) * Hkv + hk) * (D + D * D);
  for (int d = threadIdx.x; d < D; d += blockDim.x) out[d] = s_mu[d];
  const float norm = 1.f / float(max(1, rows - 1));
  // each thread owns strips of four columns of one row of Sigma
  for (int e = threadIdx.x; e < D * D / 4; e += blockDim.x) {
    const int i = e / (D / 4), j0 = (e % (D / 4)) * 4;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    for (int r = 0; r < rows; ++r) {
      const float qi = s_q[r * D + i];
      const float4 qj = *reinterpret_cast<const float4*>(&s_q[r * D + j0]);
      a0 += qi * qj.x;
      a1 += qi * qj.y;
      a2 += qi * qj.z;
      a3 += qi * qj.w;
    }
    *reinterpret_cast<float4*>(&out[D + i * D + j0]) = make_float4(a0 * norm, a1 * norm, a2 * norm, a3 * norm);
  }
}

// ------------------------------------------------------------------ scores
// grid (key tiles of EA_KEYS_PER_CTA, Hkv, n_seq * L), 256 threads.  Sigma stays in shared memory (rows padded to
// D + 4 floats: 16-byte aligned and conflict-free for 128-bit reads).  A warp takes EA_KB keys at a time: lane l owns
// rows l, l + 32, ... of Sigma and accumulates (Sigma k)_row for the EA_KB keys at once, so every 128-bit piece of a
// Sigma row read from shared memory feeds 4 * EA_KB multiply-adds (one key at a time, two shared-memory reads per
// multiply-add bound the kernel).
constexpr int EA_KEYS_PER_CTA = 512;
constexpr int EA_KB = 8;

template <int D>
__global__ void __launch_bounds__(256)
ea_scores_kernel(const bf16* __restrict__ pool, const float* __restrict__ stats, const int* __restrict__ block_tables,
                 const int* __restrict__ kv_lens, float* __restrict__ scores, int L, int num_blocks, int Hkv,
                 int block_size, int max_blocks, int stride, int n_sink, uint32_t* status) {
  constexpr int PER = D / 32;                                // Sigma rows (and key elements) per lane
  constexpr int CP = D + 4;                                  // padded row of Sigma, floats
  extern __shared__ __align__(16) uint8_t smem[];
  float* s_cov = reinterpret_cast<float*>(smem);             // [D][CP]
  float* s_mu = s_cov + D * CP;
  float* s_k = s_mu + D;                                     // [8 warps][EA_KB][D]
  const int hk = blockIdx.y, unit_sl = blockIdx.z;
  const int seq = unit_sl / L, layer = unit_sl % L;
  const int S = kv_lens[seq];
  const int c_begin = blockIdx.x * EA_KEYS_PER_CTA;
  float* out = scores + (((long long)seq * L + layer) * Hkv + hk) * stride;
  if (c_begin >= stride) return;
  const float* st = stats + (((long long)seq * L + layer) * Hkv + hk) * (D + D * D);
  if (c_begin < S) {
    for (int i = threadIdx.x; i < D * D; i += blockDim.x) s_cov[(i / D) * CP + (i % D)] = st[D + i];
    for (int i = threadIdx.x; i < D; i += blockDim.x) s_mu[i] = st[i];
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* bt = block_tables + (long long)seq * max_blocks;
  const bf16* kbase = pool + ((long long)layer * 2) * num_blocks * Hkv * block_size * D;
  const bf16* vbase = kbase + (long long)num_blocks * Hkv * block_size * D;
  const float inv_sqrt_d = rsqrtf(float(D)), inv_2d = 0.5f / float(D);
  float* myk = s_k + warp * EA_KB * D;
  const int c_end = min(c_begin + EA_KEYS_PER_CTA, stride);
  for (int c0 = c_begin + warp * EA_KB; c0 < c_end; c0 += 8 * EA_KB) {
    // ---- the keys of this group into shared memory (zeros for rows that get a fixed score)
    float vss[EA_KB], lin[EA_KB];
#pragma unroll
    for (int kb = 0; kb < EA_KB; ++kb) {
      const int c = c0 + kb;
      vss[kb] = lin[kb] = 0.f;
      const bool live = c < S && c >= n_sink;
      long long off = 0;
      if (live) {
        int blk = bt[c / block_size];
        if (blk < 0 || blk >= num_blocks) {
          report(status, ST_BAD_INDEX);
          blk = 0;
        }
        off = (((long long)blk * Hkv + hk) * block_size + c % block_size) * D;
      }
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        const int d = lane + 32 * e;
        float kv = 0.f;
        if (live) {
          kv = __bfloat162float(kbase[off + d]);
          const float v = __bfloat162float(vbase[off + d]);
          vss[kb] += v * v;
          lin[kb] += kv * s_mu[d];
        }
        myk[kb * D + d] = kv;
      }
    }
    __syncwarp();
    // ---- acc[e][kb] = (Sigma k_kb)_(lane + 32 e)
    float acc[PER][EA_KB];
#pragma unroll
    for (int e = 0; e < PER; ++e) {
#pragma unroll
      for (int kb = 0; kb < EA_KB; ++kb) acc[e][kb] = 0.f;
    }
#pragma unroll 2
    for (int d = 0; d < D; d += 4) {
      float4 r[PER];
#pragma unroll
      for (int e = 0; e < PER; ++e) r[e] = *reinterpret_cast<const float4*>(s_cov + (lane + 32 * e) * CP + d);
#pragma unroll
      for (int kb = 0; kb < EA_KB; ++kb) {
        const float4 kk = *reinterpret_cast<const float4*>(myk + kb * D + d);
#pragma unroll
        for (int e = 0; e < PER; ++e)
          acc[e][kb] += r[e].x * kk.x + r[e].y * kk.y + r[e].z * kk.z + r[e].w * kk.w;
      }
    }
    // ---- quad = k^T Sigma k, then the score of every key of the group
#pragma unroll
    for (int kb = 0; kb < EA_KB; ++kb) {
      const int c = c0 + kb;
      float quad = 0.f;
#pragma unroll
      for (int e = 0; e < PER; ++e) quad += myk[kb * D + lane + 32 * e] * acc[e][kb];
      quad = warp_sum(quad);
      const float vs = warp_sum(vss[kb]), ln = warp_sum(lin[kb]);
      float result;
      if (c >= S) result = -INFINITY;
      else if (c < n_sink) result = SC_POS;
      else result = ln * inv_sqrt_d + quad * inv_2d + 0.5f * __logf(fmaxf(vs, 1e-30f));
      if (lane == 0 && c < c_end) out[c] = result;
    }
    __syncwarp();
  }
}

// ------------------------------------------------------------------ position-only scorer
// StreamingLLM: score = position, the first n_sink rows always kept, -inf past the request
__global__ void position_scores_kernel(float* __restrict__ scores, const int* __restrict__ kv_lens,
                                       int units_per_seq, int stride, int n_sink) {
  const long long unit = blockIdx.x;
  const int S = kv_lens[unit / units_per_seq];
  float* s = scores + unit * stride;
  for (int c = threadIdx.x; c < stride; c += blockDim.x)
    s[c] = c >= S ? -INFINITY : (c < n_sink ? SC_POS : float(c));
}

void launch_expected_attention_scores(const void* pool, const void* qw, const int* block_tables, const int* kv_lens,
                                      float* stats, float* scores, int n_seq, int L, int num_blocks, int Hkv, int Hq,
                                      int block_size, int D, int max_blocks, int stride, int w, int n_sink,
                                      uint32_t* status, cudaStream_t stream) {
  if (n_seq == 0) return;
  const int rows = (Hq / Hkv) * w;
  if (Hq % Hkv != 0 || rows < 2) throw std::runtime_error("expected attention: bad head grouping or window");
  const int smem1 = (rows * D + D) * 4;
  const int smem2 = (D * (D + 4) + D + 8 * EA_KB * D) * 4;
  if (smem1 > 220 * 1024) throw std::runtime_error("expected attention: (Hq / Hkv) * window * head_dim is too large");
  dim3 g1(Hkv, L, n_seq);
  dim3 g2((stride + EA_KEYS_PER_CTA - 1) / EA_KEYS_PER_CTA, Hkv, n_seq * L);
  if (D == 128) {
    cudaFuncSetAttribute(ea_stats_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1);
    cudaFuncSetAttribute(ea_scores_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2);
    ea_stats_kernel<128><<<g1, 256, smem1, stream>>>((const bf16*)qw, stats, L, Hkv, Hq, w);
    ea_scores_kernel<128><<<g2, 256, smem2, stream>>>((const bf16*)pool, stats, block_tables, kv_lens, scores, L,
                                                       num_blocks, Hkv, block_size, max_blocks, stride, n_sink, status);
  } else if (D == 64) {
    cudaFuncSetAttribute(ea_stats_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1);
    cudaFuncSetAttribute(ea_scores_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2);
    ea_stats_kernel<64><<<g1, 256, smem1, stream>>>((const bf16*)qw, stats, L, Hkv, Hq, w);
    ea_scores_kernel<64><<<g2, 256, smem2, stream>>>((const bf16*)pool, stats, block_tables, kv_lens, scores, L,
                                                      num_blocks, Hkv, block_size, max_blocks, stride, n_sink, status);
  } else {
    throw std::runtime_error("expected attention: head_dim must be 64 or 128");
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("expected attention launch: ") + cudaGetErrorString(e));
}

void launch_position_scores(float* scores, const int* kv_lens, int n_seq, int units_per_seq, int stride, int n_sink,
                            cudaStream_t stream) {
  if (n_seq == 0) return;
  position_scores_kernel<<<n_seq * units_per_seq, 256, 0, stream>>>(scores, kv_lens, units_per_seq, stride, n_sink);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("position scores launch: ") + cudaGetErrorString(e));
}

}  // namespace fc
