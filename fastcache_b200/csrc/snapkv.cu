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
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <stdexcept>
#include <string>

#include "gemm.h"
#include "kernels.h"
#include "mma.cuh"
#include "ptx.cuh"

namespace fc {

using bf16 = __nv_bfloat16;

static int g_snap_tc = -1;
bool snapkv_tensor_cores() {
  if (g_snap_tc < 0) {
    const char* e = std::getenv("FC_SNAPKV_TC");
    g_snap_tc = (e == nullptr || e[0] != '0') ? 1 : 0;
  }
  return g_snap_tc == 1;
}
void set_snapkv_tensor_cores(bool on) { g_snap_tc = on ? 1 : 0; }

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

// ------------------------------------------------------------------ votes on tcgen05 (head_dim 128)
// The same two passes with the products on the tensor cores, one CTA per (KV head, layer, request):
//   pass 1  S = Q K^T with the G * w window rows as the 128-row operand (two MMAs for 256 rows) and a tile of 128
//           keys as N: the thread that owns a query row keeps its running maximum and sum (as in the attention
//           kernels, but nothing is written back)
//   pass 2  S^T = K Q^T with the 128 keys of a tile as the 128-row operand and the window rows as N: the thread
//           that owns a KEY sums exp2(s - m_q) / l_q over the query columns, so a key's votes need no reduction
//           across threads (the two warpgroups take half of the columns each and meet in shared memory)
// The Q tile and the K tiles (TMA through the block table, three-stage ring, 128-byte swizzle) are the same shared-
// memory tiles in both passes; only the roles of the operands change.  Accumulators: two buffers of 256 TMEM columns.
constexpr int SKT_THREADS = 320;
constexpr int SKT_STAGES = 3;
constexpr int SKT_K_BYTES = 128 * 128 * 2;          // one key tile: two [128 x 64] sub-tiles
constexpr int SKT_Q_BYTES = 256 * 128 * 2;          // up to 256 query rows: two [256 x 64] sub-tiles
constexpr int SKT_SMEM = SKT_Q_BYTES + SKT_STAGES * SKT_K_BYTES + 256 * 8 + 2 * 128 * 4 + 256 + 1024;

struct SnapTcParams {
  const int* block_tables;
  const int* kv_lens;
  float* votes;
  int L, num_blocks, Hkv, Hq, block_size, box_rows, max_blocks, stride, w, rows;
  float scale_log2;
  uint32_t* status;
};

__device__ __forceinline__ uint64_t skt_sdesc(uint32_t addr, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((addr & 0x3FFFF) >> 4);
  d |= uint64_t(1) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}
__device__ __forceinline__ void skt_bar256() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__global__ void __launch_bounds__(SKT_THREADS, 1)
snapkv_votes_tc_kernel(const __grid_constant__ CUtensorMap tm_pool, const __grid_constant__ CUtensorMap tm_q,
                       const SnapTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem;                                            // sub-tile 0 (256 rows), sub-tile 1
  uint8_t* s_k = s_q + SKT_Q_BYTES;                               // SKT_STAGES tiles
  float2* s_stat = reinterpret_cast<float2*>(s_k + SKT_STAGES * SKT_K_BYTES);     // [256] (m, 1 / l) per query row
  float* s_part = reinterpret_cast<float*>(s_stat + 256);         // [2][128] votes of the two column halves
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_part + 256);
  uint64_t* q_full = bars;                 // [1]
  uint64_t* k_full = bars + 1;             // [SKT_STAGES]
  uint64_t* k_empty = k_full + SKT_STAGES; // [SKT_STAGES]
  uint64_t* s_full = k_empty + SKT_STAGES; // [2]
  uint64_t* s_empty = s_full + 2;          // [2], 256 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_empty + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hk = blockIdx.x, layer = blockIdx.y, seq = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int S = p.kv_lens[seq];
  const int n_old = S - p.w;                                      // keys that can be evicted
  const int n1 = (S + 127) / 128;                                 // tiles of pass 1 (all keys)
  const int n2 = n_old > 0 ? (n_old + 127) / 128 : 0;             // tiles of pass 2 (keys that get votes)
  float* votes = p.votes + (((long long)seq * p.L + layer) * p.Hkv + hk) * p.stride;
  if (n_old <= 0) return;                                         // nothing to vote on (uniform over the CTA)

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < SKT_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&s_empty[b], 256);
    }
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_pool);
    tma_prefetch_desc(&tm_q);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool two_halves = p.rows > 128;

  if (warp == 0) {
    if (lane == 0) {
      // Q: CTA row (head_in_group * w + r) is window row r of query head hk * G + head_in_group
      mbar_expect_tx(q_full, uint32_t(p.rows) * 128 * 2);
      const int q_row0 = (seq * p.L + layer) * p.w;
      for (int hg = 0; hg < G; ++hg)
        for (int sub = 0; sub < 2; ++sub)
          tma_load_2d(s_q + sub * (SKT_Q_BYTES / 2) + hg * p.w * 128, &tm_q, q_full, (hk * G + hg) * 128 + sub * 64,
                      q_row0);
      const int* bt = p.block_tables + (long long)seq * p.max_blocks;
      const int pieces = 128 / p.box_rows;
      for (int i = 0; i < n1 + n2 && !*s_abort; ++i) {
        const int t = i < n1 ? i : i - n1;
        const int st = i % SKT_STAGES;
        if (!mbar_wait(&k_empty[st], ((uint32_t(i / SKT_STAGES)) & 1u) ^ 1u, p.status, ST_TIMEOUT_EMPTY)) {
          *s_abort = 1;
          break;
        }
        const int row0 = t * 128;
        uint32_t bytes = 0;
        for (int pc = 0; pc < pieces; ++pc)
          if (row0 + pc * p.box_rows < S) bytes += uint32_t(2 * p.box_rows * 128);
        mbar_expect_tx(&k_full[st], bytes);
        for (int pc = 0; pc < pieces; ++pc) {
          const int tok = row0 + pc * p.box_rows;
          if (tok >= S) break;
          int blk = bt[tok / p.block_size];
          if (blk < 0 || blk >= p.num_blocks) {
            report(p.status, ST_BAD_INDEX);
            blk = 0;
          }
          const long long grow =
              ((((long long)layer * 2) * p.num_blocks + blk) * p.Hkv + hk) * p.block_size + tok % p.block_size;
          uint8_t* dst = s_k + st * SKT_K_BYTES + pc * p.box_rows * 128;
          tma_load_2d(dst, &tm_pool, &k_full[st], 0, int(grow));
          tma_load_2d(dst + SKT_K_BYTES / 2, &tm_pool, &k_full[st], 64, int(grow));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc1 = make_idesc_bf16(128, 128);      // pass 1: 128 query rows x 128 keys
      const uint32_t idesc2 = make_idesc_bf16(128, p.rows);       // pass 2: 128 keys x all query rows
      bool ok = mbar_wait(q_full, 0, p.status, ST_TIMEOUT_FULL);
      const uint32_t qa = smem_u32(s_q);
      for (int i = 0; i < n1 + n2 && ok; ++i) {
        const int st = i % SKT_STAGES, buf = i & 1;
        if (*s_abort || !mbar_wait(&s_empty[buf], ((uint32_t(i) >> 1) & 1u) ^ 1u, p.status, ST_TIMEOUT_ACC_EMPTY) ||
            !mbar_wait(&k_full[st], (uint32_t(i / SKT_STAGES)) & 1u, p.status, ST_TIMEOUT_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t ka = smem_u32(s_k + st * SKT_K_BYTES);
        const uint32_t acc = tmem_base + uint32_t(buf * 256);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t qoff = uint32_t(kk >> 2) * (SKT_Q_BYTES / 2) + uint32_t(kk & 3) * 32;
          const uint32_t koff = uint32_t(kk >> 2) * (SKT_K_BYTES / 2) + uint32_t(kk & 3) * 32;
          if (i < n1) {
            tc_mma_f16(acc, skt_sdesc(qa + qoff, 1024), skt_sdesc(ka + koff, 1024), idesc1, kk > 0 ? 1u : 0u);
            if (two_halves)
              tc_mma_f16(acc + 128, skt_sdesc(qa + qoff + 128 * 128, 1024), skt_sdesc(ka + koff, 1024), idesc1,
                         kk > 0 ? 1u : 0u);
          } else {
            tc_mma_f16(acc, skt_sdesc(ka + koff, 1024), skt_sdesc(qa + qoff, 1024), idesc2, kk > 0 ? 1u : 0u);
          }
        }
        tc_commit(&k_empty[st]);
        tc_commit(&s_full[buf]);
      }
      if (!ok) *s_abort = 1;
    }
  } else {
    // ------------------------------------------------ the 256 threads that read the accumulators
    const int x = (warp - 2) >> 2;                           // warpgroup: query half in pass 1, column half in pass 2
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;                  // TMEM lane: query row (pass 1) or key (pass 2)
    const uint32_t lane_addr = uint32_t(lane_group * 32) << 16;
    const int qrow = x * 128 + row;                          // query row of this thread in pass 1
    const bool q_live = qrow < p.rows;
    const int qpos = n_old + qrow % p.w;                     // last key this query row may see
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int i = 0; i < n1; ++i) {
      const int buf = i & 1;
      if (ok && (*s_abort || !mbar_wait(&s_full[buf], (uint32_t(i) >> 1) & 1u, p.status, ST_TIMEOUT_ACC_FULL))) {
        ok = false;
        *s_abort = 1;
      }
      tc_fence_after();
      if (ok && q_live) {
        uint32_t s[128];
        const uint32_t ts = tmem_base + lane_addr + uint32_t(buf * 256 + x * 128);
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32x32(ts + uint32_t(c * 32), *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
        tmem_ld_wait();
        const int col0 = i * 128;
        if (col0 + 127 > qpos || col0 + 128 > S) {
#pragma unroll
          for (int t = 0; t < 128; ++t)
            if (col0 + t > qpos || col0 + t >= S) s[t] = 0xff800000u;
        }
        float mx = -INFINITY;
#pragma unroll
        for (int t = 0; t < 128; ++t) mx = fmaxf(mx, __uint_as_float(s[t]));
        mx *= p.scale_log2;
        const float m_new = fmaxf(m_run, mx);
        if (m_new > -INFINITY) {
          float rs = 0.f;
#pragma unroll
          for (int t = 0; t < 128; ++t) {
            float e;
            const float a = fmaf(__uint_as_float(s[t]), p.scale_log2, -m_new);
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(a));
            rs += e;
          }
          l_run = l_run * exp2f(m_run - m_new) + rs;
          m_run = m_new;
        }
      }
      tc_fence_before();
      mbar_arrive(&s_empty[buf]);
    }
    if (q_live) s_stat[qrow] = make_float2(m_run == -INFINITY ? 0.f : m_run, l_run > 0.f ? 1.f / l_run : 0.f);
    skt_bar256();
    // ---- pass 2: this thread owns key (tile * 128 + row) and half of the query columns
    const int half_cols = p.rows / 2;
    const float inv_rows = 1.f / float(p.rows);
    for (int j = 0; j < n2; ++j) {
      const int i = n1 + j, buf = i & 1;
      if (ok && (*s_abort || !mbar_wait(&s_full[buf], (uint32_t(i) >> 1) & 1u, p.status, ST_TIMEOUT_ACC_FULL))) {
        ok = false;
        *s_abort = 1;
      }
      tc_fence_after();
      float v = 0.f;
      if (ok) {
        const uint32_t ts = tmem_base + lane_addr + uint32_t(buf * 256 + x * half_cols);
#pragma unroll 1
        for (int c = 0; c < half_cols / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(ts + uint32_t(c * 32), r);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            const float2 st = s_stat[x * half_cols + c * 32 + t];
            float e;
            const float a = fmaf(__uint_as_float(r[t]), p.scale_log2, -st.x);
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(a));
            v = fmaf(e, st.y, v);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&s_empty[buf]);
      s_part[x * 128 + row] = v;
      skt_bar256();
      if (x == 0 && ok) {
        const int c = j * 128 + row;
        if (c < n_old) votes[c] = (s_part[row] + s_part[128 + row]) * inv_rows;
      }
      skt_bar256();                                          // s_part is rewritten by the next tile
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
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
  int box_rows = 128;
  while (box_rows > block_size || block_size % box_rows != 0) box_rows >>= 1;
  const long long pool_rows = (long long)L * 2 * num_blocks * Hkv * block_size;
  if (D == 128 && snapkv_tensor_cores() && rows % 64 == 0 && box_rows >= 8 && pool_rows < (1ll << 31) &&
      (long long)n_seq * L * w < (1ll << 31)) {
    SnapTcParams q{};
    q.block_tables = block_tables;
    q.kv_lens = kv_lens;
    q.votes = votes;
    q.L = L;
    q.num_blocks = num_blocks;
    q.Hkv = Hkv;
    q.Hq = Hq;
    q.block_size = block_size;
    q.box_rows = box_rows;
    q.max_blocks = max_blocks;
    q.stride = stride;
    q.w = w;
    q.rows = rows;
    q.scale_log2 = p.scale_log2;
    q.status = status;
    const CUtensorMap tp = make_tmap_bf16_2d(pool, (uint64_t)pool_rows, 128, 128, box_rows, 64);
    const CUtensorMap tq = make_tmap_bf16_2d(qw, (uint64_t)n_seq * L * w, (uint64_t)Hq * 128, (uint64_t)Hq * 128, w, 64);
    cudaFuncSetAttribute(snapkv_votes_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SKT_SMEM);
    // votes of requests no longer than the window are never written by the kernel and never read by the pooling
    snapkv_votes_tc_kernel<<<grid, SKT_THREADS, SKT_SMEM, stream>>>(tp, tq, q);
  } else if (D == 128) {
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
