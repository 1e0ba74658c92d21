// KV scoring kernels that need no attention pass: ExpectedAttention (query statistics) and the
// position-only StreamingLLM scorer.
//
// Scores are fp32 [n_seq, L, Hkv, stride]; the selection kernel (evict.cu) only ranks them, so the
// ExpectedAttention score is kept in the log domain:
//     log score[c] = k_c . mu / sqrt(D) + k_c^T Sigma k_c / (2 D) + log ||v_c||
// which orders the keys exactly like exp(logit - max) * ||v|| of the kvpress statement.  mu and Sigma
// are the mean and the (unbiased) covariance of the observation-window queries of the G query heads
// that share the KV head.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <stdexcept>
#include <string>

#include "gemm.h"
#include "kernels.h"
#include "ptx.cuh"

namespace fc {

using bf16 = __nv_bfloat16;

constexpr float SC_POS = 3.0e38f;

// ------------------------------------------------------------------ query statistics
// grid (Hkv, L, n_seq), 256 threads.  stats[unit] = mu[D] followed by Sigma[D][D].
// The G * w window rows of the KV head stay in shared memory as bf16 (64 KB for 256 x 128: three CTAs share an
// SM).  Sigma = (Q^T Q - rows mu mu^T) / (rows - 1) with fp32 sums; each thread owns 4 x 4 tiles of Q^T Q, so two
// 64-bit shared-memory reads feed 16 multiply-adds per query row.
template <int D>
__global__ void __launch_bounds__(256)
ea_stats_kernel(const bf16* __restrict__ qw, float* __restrict__ stats, bf16* __restrict__ sig16, int L, int Hkv,
                int Hq, int w) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int hk = blockIdx.x, layer = blockIdx.y, seq = blockIdx.z;
  const int G = Hq / Hkv, rows = G * w;
  bf16* s_q = reinterpret_cast<bf16*>(smem);                 // [rows][D]
  float* s_mu = reinterpret_cast<float*>(s_q + rows * D);    // [D]
  float* s_half = s_mu + D;                                  // [256 / D][D] partial column sums
  const bf16* src = qw + (((long long)seq * L + layer) * w) * Hq * D;
  constexpr int CH = D / 8;                                  // 16-byte pieces per row
  for (int i = threadIdx.x; i < rows * CH; i += blockDim.x) {
    const int r = i / CH, ch = i % CH;
    const int hg = r / w, wr = r % w;
    *reinterpret_cast<uint4*>(s_q + r * D + ch * 8) =
        *reinterpret_cast<const uint4*>(src + ((long long)wr * Hq + hk * G + hg) * D + ch * 8);
  }
  __syncthreads();
  {
    // column sums: thread (part, d) adds every (256 / D)-th row
    const int d = threadIdx.x % D, part = threadIdx.x / D, parts = blockDim.x / D;
    float acc = 0.f;
    for (int r = part; r < rows; r += parts) acc += __bfloat162float(s_q[r * D + d]);
    s_half[part * D + d] = acc;
    __syncthreads();
    if (threadIdx.x < D) {
      float tot = 0.f;
      for (int q = 0; q < parts; ++q) tot += s_half[q * D + threadIdx.x];
      s_mu[threadIdx.x] = tot / float(rows);
    }
    __syncthreads();
  }
  float* out = stats + (((long long)seq * L + layer) * Hkv + hk) * (D + D * D);
  for (int d = threadIdx.x; d < D; d += blockDim.x) out[d] = s_mu[d];
  const float norm = 1.f / float(max(1, rows - 1)), frows = float(rows);
  for (int e = threadIdx.x; e < (D / 4) * (D / 4); e += blockDim.x) {
    const int i0 = (e / (D / 4)) * 4, j0 = (e % (D / 4)) * 4;
    float a[4][4];
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) a[x][y] = 0.f;
#pragma unroll 4
    for (int r = 0; r < rows; ++r) {
      const uint2 ri = *reinterpret_cast<const uint2*>(s_q + r * D + i0);
      const uint2 rj = *reinterpret_cast<const uint2*>(s_q + r * D + j0);
      // a bf16 is the upper half of the fp32 with the same value
      const float vi[4] = {__uint_as_float(ri.x << 16), __uint_as_float(ri.x & 0xffff0000u),
                           __uint_as_float(ri.y << 16), __uint_as_float(ri.y & 0xffff0000u)};
      const float vj[4] = {__uint_as_float(rj.x << 16), __uint_as_float(rj.x & 0xffff0000u),
                           __uint_as_float(rj.y << 16), __uint_as_float(rj.y & 0xffff0000u)};
#pragma unroll
      for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) a[x][y] = fmaf(vi[x], vj[y], a[x][y]);
    }
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int i = i0 + x;
      float v4[4];
#pragma unroll
      for (int y = 0; y < 4; ++y) v4[y] = (a[x][y] - frows * s_mu[i] * s_mu[j0 + y]) * norm;
      *reinterpret_cast<float4*>(&out[D + i * D + j0]) = make_float4(v4[0], v4[1], v4[2], v4[3]);
      if (sig16 != nullptr) {
        // Sigma as the sum of two bf16 matrices (hi + lo), for the tensor-core scoring kernel: [unit][2][D][D]
        bf16* hi = sig16 + (((long long)seq * L + layer) * Hkv + hk) * (2 * D * D) + i * D + j0;
        bf16* lo = hi + D * D;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const bf16 h = __float2bfloat16(v4[t]);
          hi[t] = h;
          lo[t] = __float2bfloat16(v4[t] - __bfloat162float(h));
        }
      }
    }
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

// ------------------------------------------------------------------ scores on tcgen05 (head_dim 128)
// Y = K Sigma for a tile of 128 keys is a [128 x 128] x [128 x 128] product: the key tile (TMA through the block
// table, 128-byte swizzle) is the A operand, Sigma the B operand (it is symmetric, so its rows serve as the K-major
// "N x K" matrix), the accumulator sits in tensor memory.  Sigma is given as hi + lo bf16 matrices (two MMAs per
// K step), which keeps the quadratic form at fp32-level accuracy although the operands are bf16.  The epilogue
// thread of a key reads its row of Y from tensor memory and its k and v rows from the same shared-memory tiles
// and finishes k.Y, k.mu and ||v||^2.  grid (chunks of EAT_TILES key tiles, Hkv, n_seq * L); two stages of K / V
// tiles and two accumulators, so the loads and MMAs of one tile run under the epilogue of the one before.
constexpr int EAT_TILES = 8;
constexpr int EAT_THREADS = 192;
constexpr int EAT_TILE_BYTES = 128 * 128 * 2;      // two [128 x 64] sub-tiles
constexpr int EAT_SUB_BYTES = EAT_TILE_BYTES / 2;
constexpr int EAT_SMEM = 2 * EAT_TILE_BYTES + 4 * EAT_TILE_BYTES + 512 + 256 + 1024;

struct EaTcParams {
  const float* stats;          // [unit][D + D * D]: mu first
  const int* block_tables;
  const int* kv_lens;
  float* scores;
  int L, num_blocks, Hkv, block_size, box_rows, max_blocks, stride, n_sink;
  uint32_t* status;
};

__global__ void __launch_bounds__(EAT_THREADS, 1)
ea_scores_tc_kernel(const __grid_constant__ CUtensorMap tm_pool, const __grid_constant__ CUtensorMap tm_sig,
                    const EaTcParams p) {
  constexpr int D = 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_sig = smem;                               // hi (2 sub-tiles), lo (2 sub-tiles)
  uint8_t* s_k = s_sig + 2 * EAT_TILE_BYTES;           // 2 stages
  uint8_t* s_v = s_k + 2 * EAT_TILE_BYTES;             // 2 stages
  float* s_mu = reinterpret_cast<float*>(s_v + 2 * EAT_TILE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_mu + D);
  uint64_t* sig_full = bars;          // [1]
  uint64_t* kv_full = bars + 1;       // [2]
  uint64_t* kv_empty = bars + 3;      // [2], 128 arrivals: the epilogue has read the tiles and the accumulator
  uint64_t* acc_full = bars + 5;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hk = blockIdx.y, unit_sl = blockIdx.z;
  const int seq = unit_sl / p.L, layer = unit_sl % p.L;
  const long long unit = ((long long)seq * p.L + layer) * p.Hkv + hk;
  const int S = p.kv_lens[seq];
  const int c_begin = blockIdx.x * EAT_TILES * 128;
  float* out = p.scores + unit * p.stride;
  if (c_begin >= p.stride) return;
  const int c_end = min(c_begin + EAT_TILES * 128, p.stride);
  if (c_begin >= S) {                                  // nothing stored here: fixed scores, no tiles
    for (int c = c_begin + threadIdx.x; c < c_end; c += EAT_THREADS) out[c] = -INFINITY;
    return;
  }
  const int n_tiles = (min(c_end, S) - c_begin + 127) / 128;
  // columns past the last tile that holds keys
  for (int c = c_begin + n_tiles * 128 + threadIdx.x; c < c_end; c += EAT_THREADS) out[c] = -INFINITY;

  if (threadIdx.x == 0) {
    mbar_init(sig_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 128);
      mbar_init(&acc_full[s], 1);
    }
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_pool);
    tma_prefetch_desc(&tm_sig);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  for (int d = threadIdx.x; d < D; d += EAT_THREADS) s_mu[d] = p.stats[unit * (D + D * D) + d];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(sig_full, 2 * EAT_TILE_BYTES);
      for (int q = 0; q < 2; ++q)                       // hi, lo: rows (unit * 2 + q) * 128 ...
        for (int sub = 0; sub < 2; ++sub)
          tma_load_2d(s_sig + q * EAT_TILE_BYTES + sub * EAT_SUB_BYTES, &tm_sig, sig_full, sub * 64,
                      int((unit * 2 + q) * D));
      const int* bt = p.block_tables + (long long)seq * p.max_blocks;
      const int pieces = 128 / p.box_rows;
      for (int t = 0; t < n_tiles && !*s_abort; ++t) {
        const int st = t & 1;
        if (!mbar_wait(&kv_empty[st], ((uint32_t(t) >> 1) & 1u) ^ 1u, p.status, ST_TIMEOUT_EMPTY)) {
          *s_abort = 1;
          break;
        }
        const int row0 = c_begin + t * 128;
        uint32_t bytes = 0;
        for (int pc = 0; pc < pieces; ++pc)
          if (row0 + pc * p.box_rows < S) bytes += uint32_t(2 * 2 * p.box_rows * 128);     // K and V, two sub-tiles
        mbar_expect_tx(&kv_full[st], bytes);
        for (int pc = 0; pc < pieces; ++pc) {
          const int tok = row0 + pc * p.box_rows;
          if (tok >= S) break;
          int blk = bt[tok / p.block_size];
          if (blk < 0 || blk >= p.num_blocks) {
            report(p.status, ST_BAD_INDEX);
            blk = 0;
          }
          for (int kv = 0; kv < 2; ++kv) {
            const long long grow =
                ((((long long)layer * 2 + kv) * p.num_blocks + blk) * p.Hkv + hk) * p.block_size + tok % p.block_size;
            uint8_t* dst = (kv == 0 ? s_k : s_v) + st * EAT_TILE_BYTES + pc * p.box_rows * 128;
            tma_load_2d(dst, &tm_pool, &kv_full[st], 0, int(grow));
            tma_load_2d(dst + EAT_SUB_BYTES, &tm_pool, &kv_full[st], 64, int(grow));
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, 128);
      bool ok = mbar_wait(sig_full, 0, p.status, ST_TIMEOUT_FULL);
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int st = t & 1;
        // kv_full[st] of tile t implies that the epilogue of tile t - 2 has released accumulator st as well
        if (*s_abort || !mbar_wait(&kv_full[st], (uint32_t(t) >> 1) & 1u, p.status, ST_TIMEOUT_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t ka = smem_u32(s_k + st * EAT_TILE_BYTES), sa = smem_u32(s_sig);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = uint32_t(kk >> 2) * EAT_SUB_BYTES + uint32_t(kk & 3) * 32;
            tc_mma_f16(tmem_base + uint32_t(st * 128), make_sdesc_sw128(ka + off),
                       make_sdesc_sw128(sa + q * EAT_TILE_BYTES + off), idesc, (q > 0 || kk > 0) ? 1u : 0u);
          }
        }
        tc_commit(&acc_full[st]);
      }
      if (!ok) *s_abort = 1;
    }
  } else {
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;
    const float inv_sqrt_d = rsqrtf(float(D)), inv_2d = 0.5f / float(D);
    bool ok = true;
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int st = t & 1;
      if (*s_abort || !mbar_wait(&acc_full[st], (uint32_t(t) >> 1) & 1u, p.status, ST_TIMEOUT_ACC_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (uint32_t(lane_group * 32) << 16) + uint32_t(st * 128);
      const uint8_t* krow = s_k + st * EAT_TILE_BYTES + row * 128;
      const uint8_t* vrow = s_v + st * EAT_TILE_BYTES + row * 128;
      const int c = c_begin + t * 128 + row;
      const bool live = c < S && c >= p.n_sink;
      float quad = 0.f, lin = 0.f, vss = 0.f;
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {                  // 32 columns of Y at a time
        uint32_t y[32];
        tmem_ld_32x32(t_addr + uint32_t(ch * 32), y);
        tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {                 // 8 elements = one 16-byte piece of the swizzled row
            const int d0 = ch * 32 + g * 8;
            const int piece = ((d0 & 63) >> 3) ^ (row & 7);
            const int offs = (d0 >> 6) * EAT_SUB_BYTES + piece * 16;
            const uint4 kq = *reinterpret_cast<const uint4*>(krow + offs);
            const uint4 vq = *reinterpret_cast<const uint4*>(vrow + offs);
            const uint32_t kw[4] = {kq.x, kq.y, kq.z, kq.w}, vw[4] = {vq.x, vq.y, vq.z, vq.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float k0 = __uint_as_float(kw[e] << 16), k1 = __uint_as_float(kw[e] & 0xffff0000u);
              const float v0 = __uint_as_float(vw[e] << 16), v1 = __uint_as_float(vw[e] & 0xffff0000u);
              quad = fmaf(k0, __uint_as_float(y[g * 8 + 2 * e]), quad);
              quad = fmaf(k1, __uint_as_float(y[g * 8 + 2 * e + 1]), quad);
              lin = fmaf(k0, s_mu[d0 + 2 * e], lin);
              lin = fmaf(k1, s_mu[d0 + 2 * e + 1], lin);
              vss = fmaf(v0, v0, vss);
              vss = fmaf(v1, v1, vss);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&kv_empty[st]);
      if (c < c_end) {
        float result;
        if (c >= S) result = -INFINITY;
        else if (c < p.n_sink) result = SC_POS;
        else result = lin * inv_sqrt_d + quad * inv_2d + 0.5f * __logf(fmaxf(vss, 1e-30f));
        out[c] = result;
      }
    }
    if (!ok) *s_abort = 1;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
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

static int g_ea_tc = -1;
bool ea_tensor_cores() {
  if (g_ea_tc < 0) {
    const char* e = std::getenv("FC_EA_TC");
    g_ea_tc = (e == nullptr || e[0] != '0') ? 1 : 0;
  }
  return g_ea_tc == 1;
}
void set_ea_tensor_cores(bool on) { g_ea_tc = on ? 1 : 0; }

// `sig16`: bf16 scratch [n_seq * L * Hkv][2][D][D] for the tensor-core form (head_dim 128), or nullptr
void launch_expected_attention_scores(const void* pool, const void* qw, const int* block_tables, const int* kv_lens,
                                      float* stats, float* scores, int n_seq, int L, int num_blocks, int Hkv, int Hq,
                                      int block_size, int D, int max_blocks, int stride, int w, int n_sink,
                                      uint32_t* status, cudaStream_t stream, void* sig16) {
  if (n_seq == 0) return;
  const int rows = (Hq / Hkv) * w;
  if (Hq % Hkv != 0 || rows < 2) throw std::runtime_error("expected attention: bad head grouping or window");
  const int smem1 = rows * D * 2 + D * 4 + 256 * 4;
  const int smem2 = (D * (D + 4) + D + 8 * EA_KB * D) * 4;
  if (smem1 > 220 * 1024) throw std::runtime_error("expected attention: (Hq / Hkv) * window * head_dim is too large");
  dim3 g1(Hkv, L, n_seq);
  dim3 g2((stride + EA_KEYS_PER_CTA - 1) / EA_KEYS_PER_CTA, Hkv, n_seq * L);
  int box_rows = 128;
  while (box_rows > block_size || block_size % box_rows != 0) box_rows >>= 1;
  const long long pool_rows = (long long)L * 2 * num_blocks * Hkv * block_size;
  const bool tc = D == 128 && sig16 != nullptr && ea_tensor_cores() && box_rows >= 8 && pool_rows < (1ll << 31) &&
                  (long long)n_seq * L * Hkv * 2 * D < (1ll << 31);
  if (D == 128) {
    cudaFuncSetAttribute(ea_stats_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1);
    ea_stats_kernel<128><<<g1, 256, smem1, stream>>>((const bf16*)qw, stats, tc ? (bf16*)sig16 : nullptr, L, Hkv, Hq, w);
    if (tc) {
      EaTcParams p{};
      p.stats = stats;
      p.block_tables = block_tables;
      p.kv_lens = kv_lens;
      p.scores = scores;
      p.L = L;
      p.num_blocks = num_blocks;
      p.Hkv = Hkv;
      p.block_size = block_size;
      p.box_rows = box_rows;
      p.max_blocks = max_blocks;
      p.stride = stride;
      p.n_sink = n_sink;
      p.status = status;
      const CUtensorMap tp = make_tmap_bf16_2d(pool, (uint64_t)pool_rows, D, D, box_rows, 64);
      const CUtensorMap ts = make_tmap_bf16_2d(sig16, (uint64_t)n_seq * L * Hkv * 2 * D, D, D, 128, 64);
      cudaFuncSetAttribute(ea_scores_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, EAT_SMEM);
      dim3 g3((stride + EAT_TILES * 128 - 1) / (EAT_TILES * 128), Hkv, n_seq * L);
      ea_scores_tc_kernel<<<g3, EAT_THREADS, EAT_SMEM, stream>>>(tp, ts, p);
    } else {
      cudaFuncSetAttribute(ea_scores_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2);
      ea_scores_kernel<128><<<g2, 256, smem2, stream>>>((const bf16*)pool, stats, block_tables, kv_lens, scores, L,
                                                         num_blocks, Hkv, block_size, max_blocks, stride, n_sink, status);
    }
  } else if (D == 64) {
    cudaFuncSetAttribute(ea_stats_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1);
    cudaFuncSetAttribute(ea_scores_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2);
    ea_stats_kernel<64><<<g1, 256, smem1, stream>>>((const bf16*)qw, stats, nullptr, L, Hkv, Hq, w);
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
