// SnapKV scores in the pool: how much the last `w` queries of a request (its observation window)
// attend to every earlier key, per KV head.
//
//   votes[c]  = mean over the G query heads of the KV head and the w window rows of
//               softmax_c(q_r . k_c / sqrt(D))  with the causal mask c <= S - w + r,   c < S - w
//   score[c]  = average of votes over a window of `kernel_size` keys (zero padding, padded count),
//               +inf-like for the window rows themselves (always kept), -inf past the request
//
// One CTA per (KV head, layer, request): all G * w query rows sit in shared memory (16 rows per warp),
// the keys are read through the block table in tiles of 64 rows (cp.async, double-buffered, swizzled)
// and walked twice: pass 1 gets each row's maximum and sum with the online recurrence, pass 2
// recomputes the scores, normalises them and sums the tile's columns over all rows (registers ->
// quad shuffles -> one shared-memory slot per warp -> fixed-order sum, so the result is deterministic).
// S = Q K^T runs on mma.sync.m16n8k16 (bf16 in, fp32 accumulate); the op is a thin GEMM, a few
// hundred MFLOP per CTA, and is bound by the second read of K.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

#include "kernels.h"
#include "mma.cuh"
#include "ptx.cuh"

namespace fc {

using bf16 = __nv_bfloat16;

constexpr int SK_TILE = 64;        // keys per tile
constexpr float SK_POS = 3.0e38f;  // score of the rows that are always kept

struct SnapParams {
  const bf16* pool;                // [L, 2, NB, Hkv, bs, D]
  const bf16* qw;                  // [n_seq, L, w, Hq, D]
  const int* block_tables;         // [n_seq, max_blocks]
  const int* kv_lens;              // [n_seq]
  float* votes;                    // [n_seq, L, Hkv, stride] raw votes
  int L, num_blocks, Hkv, Hq, block_size, max_blocks, stride, w;
  float scale_log2;
  uint32_t* status;
};

template <int D>
__global__ void __launch_bounds__(512)
snapkv_votes_kernel(const SnapParams p) {
  constexpr int CH = D / 8;
  constexpr int T_BYTES = SK_TILE * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const int hk = blockIdx.x, layer = blockIdx.y, seq = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int rows = G * p.w;                                  // query rows of this CTA, 16 per warp
  const int warps = rows / 16;
  const uint32_t s_q = smem_u32(smem);
  const uint32_t s_k = s_q + rows * D * 2;                   // two stages
  float* s_red = reinterpret_cast<float*>(smem + rows * D * 2 + 2 * T_BYTES);   // [warps][SK_TILE]

  const int S = p.kv_lens[seq];
  const int n_old = S - p.w;                                 // keys that can be evicted
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int* bt = p.block_tables + (long long)seq * p.max_blocks;
  const bf16* kbase = p.pool + ((long long)layer * 2) * p.num_blocks * p.Hkv * p.block_size * D;
  float* votes = p.votes + (((long long)seq * p.L + layer) * p.Hkv + hk) * p.stride;
  const int n_tiles = (S + SK_TILE - 1) / SK_TILE;

  // ---- Q rows -> smem: CTA row (head_in_group * w + r) is window row r of query head hk * G + head_in_group
  const bf16* qsrc = p.qw + (((long long)seq * p.L + layer) * p.w) * p.Hq * D;
  for (int c = threadIdx.x; c < rows * CH; c += blockDim.x) {
    const int r = c / CH, ch = c % CH;
    const int hg = r / p.w, wr = r % p.w;
    cp_async16(s_q + swz<D>(r, ch), qsrc + ((long long)wr * p.Hq + hk * G + hg) * D + ch * 8, true);
  }
  auto load_tile = [&](int tile, int stage) {
    const uint32_t sk = s_k + stage * T_BYTES;
    const int row0 = tile * SK_TILE;
    for (int c = threadIdx.x; c < SK_TILE * CH; c += blockDim.x) {
      const int r = c / CH, ch = c % CH;
      const int tok = row0 + r;
      bool valid = tok < S;
      long long off = 0;
      if (valid) {
        const int blk = bt[tok / p.block_size];
        if (blk < 0 || blk >= p.num_blocks) {
          report(p.status, ST_BAD_INDEX);
          valid = false;
        } else {
          off = (((long long)blk * p.Hkv + hk) * p.block_size + tok % p.block_size) * D + ch * 8;
        }
      }
      cp_async16(sk + swz<D>(r, ch), kbase + off, valid);
    }
  };

  uint32_t qa[D / 16][4];
  const int wr0 = (warp * 16 + g) % p.w;                     // window row of this thread's first row (w % 16 == 0)
  const int qpos0 = n_old + wr0, qpos1 = qpos0 + 8;          // last key each row may see
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float inv0 = 0.f, inv1 = 0.f;

  for (int pass = 0; pass < 2; ++pass) {
    load_tile(0, 0);
    cp_async_commit();
    for (int it = 0; it < n_tiles; ++it) {
      if (it + 1 < n_tiles) load_tile(it + 1, (it + 1) & 1);
      cp_async_commit();
      cp_async_wait<1>();
      __syncthreads();
      if (pass == 0 && it == 0) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const int mat = lane >> 3;
          const int r = warp * 16 + (mat & 1) * 8 + (lane & 7);
          const int ch = kk * 2 + (mat >> 1);
          ldsm_x4(s_q + swz<D>(r, ch), qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
        }
      }
      const uint32_t sk = s_k + (it & 1) * T_BYTES;
      float sc[SK_TILE / 8][4];
#pragma unroll
      for (int n = 0; n < SK_TILE / 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < SK_TILE / 16; ++np) {
          const int mat = lane >> 3;
          const int r = np * 16 + (mat >> 1) * 8 + (lane & 7);
          const int ch = kk * 2 + (mat & 1);
          uint32_t b0, b1, b2, b3;
          ldsm_x4(sk + swz<D>(r, ch), b0, b1, b2, b3);
          mma_bf16(sc[2 * np], qa[kk], b0, b1);
          mma_bf16(sc[2 * np + 1], qa[kk], b2, b3);
        }
      }
      const int col0 = it * SK_TILE;
      const bool need_mask = col0 + SK_TILE > n_old;          // only the last tiles touch the window / the end
      if (pass == 0) {
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < SK_TILE / 8; ++n) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = col0 + n * 8 + 2 * t + e;
            float a = sc[n][e] * p.scale_log2, b = sc[n][2 + e] * p.scale_log2;
            if (need_mask) {
              if (col > qpos0) a = -INFINITY;
              if (col > qpos1) b = -INFINITY;
            }
            sc[n][e] = a;
            sc[n][2 + e] = b;
            mx0 = fmaxf(mx0, a);
            mx1 = fmaxf(mx1, b);
          }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
        const float base0 = (nm0 == -INFINITY) ? 0.f : nm0, base1 = (nm1 == -INFINITY) ? 0.f : nm1;
        float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
        for (int n = 0; n < SK_TILE / 8; ++n) {
          rs0 += exp2f(sc[n][0] - base0) + exp2f(sc[n][1] - base0);
          rs1 += exp2f(sc[n][2] - base1) + exp2f(sc[n][3] - base1);
        }
        l0 = l0 * exp2f(m0 - base0) + rs0;
        l1 = l1 * exp2f(m1 - base1) + rs1;
        m0 = nm0;
        m1 = nm1;
      } else if (col0 < n_old) {
        // normalised probabilities of this tile, summed over the 16 rows of the warp
#pragma unroll
        for (int n = 0; n < SK_TILE / 8; ++n) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = col0 + n * 8 + 2 * t + e;
            float a = exp2f(sc[n][e] * p.scale_log2 - m0) * inv0;
            float b = exp2f(sc[n][2 + e] * p.scale_log2 - m1) * inv1;
            if (need_mask) {
              if (col > qpos0) a = 0.f;
              if (col > qpos1) b = 0.f;
            }
            float v = a + b;
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            if (g == 0) s_red[warp * SK_TILE + n * 8 + 2 * t + e] = v;
          }
        }
        __syncthreads();
        for (int c = threadIdx.x; c < SK_TILE; c += blockDim.x) {
          float tot = 0.f;
          for (int w2 = 0; w2 < warps; ++w2) tot += s_red[w2 * SK_TILE + c];
          if (col0 + c < n_old) votes[col0 + c] = tot / float(rows);
        }
      }
      __syncthreads();                                       // stage (it & 1) and s_red may be rewritten
    }
    cp_async_wait<0>();
    if (pass == 0) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
      l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
      l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
      l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
      inv0 = l0 > 0.f ? 1.f / l0 : 0.f;
      inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
      if (m0 == -INFINITY) m0 = 0.f;
      if (m1 == -INFINITY) m1 = 0.f;
    }
  }
}

// scores[c] = mean of votes[c - k/2 .. c + k/2] (zeros outside [0, n_old), divided by k); window rows
// get SK_POS, columns past the request -inf
__global__ void snapkv_pool_kernel(const float* __restrict__ votes, float* __restrict__ scores,
                                   const int* __restrict__ kv_lens, int units_per_seq, int stride, int w,
                                   int kernel_size) {
  const long long unit = blockIdx.x;
  const int S = kv_lens[unit / units_per_seq];
  const int n_old = S - w;
  const float* v = votes + unit * stride;
  float* s = scores + unit * stride;
  const int half = kernel_size / 2;
  for (int c = threadIdx.x; c < stride; c += blockDim.x) {
    float out;
    if (c >= S) {
      out = -INFINITY;
    } else if (c >= n_old) {
      out = SK_POS;
    } else if (kernel_size > 1) {
      float acc = 0.f;
      for (int d = -half; d <= half; ++d) {
        const int cc = c + d;
        if (cc >= 0 && cc < n_old) acc += v[cc];
      }
      out = acc / float(kernel_size);
    } else {
      out = v[c];
    }
    s[c] = out;
  }
}

void launch_snapkv_scores(const void* pool, const void* qw, const int* block_tables, const int* kv_lens, float* votes,
                          float* scores, int n_seq, int L, int num_blocks, int Hkv, int Hq, int block_size, int D,
                          int max_blocks, int stride, int w, int kernel_size, float scale, uint32_t* status,
                          cudaStream_t stream) {
  if (n_seq == 0) return;
  const int G = Hq / Hkv, rows = G * w;
  if (Hq % Hkv != 0 || w % 16 != 0 || rows > 256 || rows < 16)
    throw std::runtime_error("snapkv scores: window must be a multiple of 16 and (Hq / Hkv) * window <= 256");
  if (kernel_size % 2 == 0) throw std::runtime_error("snapkv scores: the pooling kernel must be odd");
  SnapParams p{};
  p.pool = reinterpret_cast<const bf16*>(pool);
  p.qw = reinterpret_cast<const bf16*>(qw);
  p.block_tables = block_tables;
  p.kv_lens = kv_lens;
  p.votes = votes;
  p.L = L;
  p.num_blocks = num_blocks;
  p.Hkv = Hkv;
  p.Hq = Hq;
  p.block_size = block_size;
  p.max_blocks = max_blocks;
  p.stride = stride;
  p.w = w;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  const int warps = rows / 16;
  const int smem = rows * D * 2 + 2 * SK_TILE * D * 2 + warps * SK_TILE * 4;
  dim3 grid(Hkv, L, n_seq);
  if (D == 128) {
    cudaFuncSetAttribute(snapkv_votes_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    snapkv_votes_kernel<128><<<grid, warps * 32, smem, stream>>>(p);
  } else if (D == 64) {
    cudaFuncSetAttribute(snapkv_votes_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    snapkv_votes_kernel<64><<<grid, warps * 32, smem, stream>>>(p);
  } else {
    throw std::runtime_error("snapkv scores: head_dim must be 64 or 128");
  }
  snapkv_pool_kernel<<<n_seq * L * Hkv, 256, 0, stream>>>(votes, scores, kv_lens, L * Hkv, stride, w, kernel_size);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("snapkv scores launch: ") + cudaGetErrorString(e));
}

}  // namespace fc
