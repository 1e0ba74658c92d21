// Causal prefill attention on tcgen05, head_dim 128: two query tiles per CTA in ping-pong.
//
// One CTA owns 256 query rows of one head (tiles A and B of 128 rows) and walks the visible keys
// in tiles of 128 rows.  All accumulators live in tensor memory (512 columns):
//     S_A [0,128)  S_B [128,256)  O_A [256,384)  O_B [384,512)
//   warp 0       TMA: both Q tiles once, then K and V tiles (boxes that never straddle a pool
//                block) into 2-stage rings, 128-byte swizzle
//   warp 1       tcgen05.mma issuer.  S_X = Q_X K^T (operands from shared memory).  O_X += P_X V with
//                P_X read from TENSOR MEMORY (it overwrites the first 64 columns of S_X as packed
//                bf16) and V as an MN-major shared-memory operand.  The issue order
//                PV_A(j) S_A(j+1) PV_B(j) S_B(j+1) keeps the tensor core busy with one tile's
//                matrices while the other tile's softmax runs.
//   warps 2-5    softmax of tile A, warps 6-9 of tile B: one query row per thread; the row of S is
//                read once into registers, exponentiated against a reference maximum and written
//                back as P.  O is rescaled only when a row maximum grows by more than 2^8 over the
//                reference (all lanes of the warp then rescale their O row in tensor memory), so
//                most tiles never touch O; the reference maximum cancels in O / l at the end.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

#include "gemm.h"
#include "kernels.h"
#include "ptx.cuh"

namespace fc {

using bf16 = __nv_bfloat16;

constexpr int P2_BM = 128;             // rows per query tile (two tiles per CTA)
constexpr int P2_BN = 128;
constexpr int P2_D = 128;
constexpr int P2_THREADS = 320;
constexpr int P2_TILE_BYTES = P2_BN * P2_D * 2;        // 32 KiB: two [128 x 64] sub-tiles
constexpr int P2_SUB_BYTES = P2_TILE_BYTES / 2;
constexpr float P2_RESCALE_THRESHOLD = 8.f;            // log2 units

__device__ __forceinline__ uint64_t p2_sdesc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((addr & 0x3FFFF) >> 4);
  d |= uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}

struct PrefillTc2Params {
  const int* block_tables;
  const int* cu_q;
  const int* kv_lens;
  bf16* out;
  int Hq, Hkv, block_size, box_rows, max_blocks, num_blocks;
  float scale_log2;
  uint32_t* status;
};

__global__ void __launch_bounds__(P2_THREADS, 1)
prefill_attn_tc2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const PrefillTc2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem;                                   // 2 tiles
  uint8_t* s_k = s_q + 2 * P2_TILE_BYTES;                // 2 stages
  uint8_t* s_v = s_k + 2 * P2_TILE_BYTES;                // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_v + 2 * P2_TILE_BYTES);
  uint64_t* q_full = bars;            // [1]
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [2] per query tile
  uint64_t* p_ready = bars + 11;      // [2] per query tile (128 arrivals)
  uint64_t* o_done = bars + 13;       // [2] per query tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.z, h = blockIdx.y;
  const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_begin;
  const int q0 = (gridDim.x - 1 - blockIdx.x) * (2 * P2_BM);        // late (long) tiles first
  if (q0 >= q_len) return;
  const int kv_len = p.kv_lens[seq];
  const int offset = kv_len - q_len;
  const int hk = h / (p.Hq / p.Hkv);
  const bool act_b = q0 + P2_BM < q_len;
  // keys visible to each query tile, in tiles of 128
  const int kv_end_a = min(kv_len, offset + q0 + P2_BM);
  const int kv_end_b = act_b ? min(kv_len, offset + q0 + 2 * P2_BM) : 0;
  const int n_a = (kv_end_a + P2_BN - 1) / P2_BN;
  const int n_b = (kv_end_b + P2_BN - 1) / P2_BN;
  const int n_tiles = max(n_a, n_b);
  const int kv_end = max(kv_end_a, kv_end_b);
  const int* bt = p.block_tables + (long long)seq * p.max_blocks;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_ready[s], 128);
      mbar_init(&o_done[s], 1);
    }
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  // V rows past the visible keys are never loaded; 0 * (uninitialised bits) must not produce NaN
  for (int i = threadIdx.x; i < 2 * P2_TILE_BYTES / 16; i += P2_THREADS)
    reinterpret_cast<uint4*>(s_v)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async();
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA loader
    if (lane == 0) {
      mbar_expect_tx(q_full, (act_b ? 2 : 1) * P2_TILE_BYTES);
      for (int x = 0; x < (act_b ? 2 : 1); ++x) {
        tma_load_2d(s_q + x * P2_TILE_BYTES, &tm_q, q_full, h * P2_D, q_begin + q0 + x * P2_BM);
        tma_load_2d(s_q + x * P2_TILE_BYTES + P2_SUB_BYTES, &tm_q, q_full, h * P2_D + 64, q_begin + q0 + x * P2_BM);
      }
      const int pieces = P2_BN / p.box_rows;
      for (int j = 0; j < n_tiles && !*s_abort; ++j) {
        const int st = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        const int row0 = j * P2_BN;
        uint32_t bytes = 0;
        for (int pc = 0; pc < pieces; ++pc)
          if (row0 + pc * p.box_rows < kv_end) bytes += uint32_t(2 * p.box_rows * 128);
        for (int which = 0; which < 2; ++which) {
          uint64_t* full = which == 0 ? &k_full[st] : &v_full[st];
          uint64_t* empty = which == 0 ? &k_empty[st] : &v_empty[st];
          if (!mbar_wait(empty, ph, p.status, ST_TIMEOUT_EMPTY)) {
            *s_abort = 1;
            break;
          }
          uint8_t* dst = (which == 0 ? s_k : s_v) + st * P2_TILE_BYTES;
          mbar_expect_tx(full, bytes);
          for (int pc = 0; pc < pieces; ++pc) {
            const int tok = row0 + pc * p.box_rows;
            if (tok >= kv_end) break;
            int blk = bt[tok / p.block_size];
            if (blk < 0 || blk >= p.num_blocks) {
              report(p.status, ST_BAD_INDEX);
              blk = 0;
            }
            const int grow = (blk * p.Hkv + hk) * p.block_size + tok % p.block_size;
            const CUtensorMap* tm = which == 0 ? &tm_k : &tm_v;
            tma_load_2d(dst + pc * p.box_rows * 128, tm, full, 0, grow);
            tma_load_2d(dst + P2_SUB_BYTES + pc * p.box_rows * 128, tm, full, 64, grow);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, false, true);    // B (= V) is MN-major
      bool ok = mbar_wait(q_full, 0, p.status, ST_TIMEOUT_FULL);
      // S_x(j) = Q_x K(j)^T into tensor-memory columns [x * 128, x * 128 + 128)
      auto issue_s = [&](int x, int j) {
        const int st = j & 1;
        const uint32_t qa = smem_u32(s_q + x * P2_TILE_BYTES), ka = smem_u32(s_k + st * P2_TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = uint32_t(kk >> 2) * P2_SUB_BYTES + uint32_t(kk & 3) * 32;
          tc_mma_f16(tmem_base + uint32_t(x * 128), p2_sdesc(qa + off, 16, 1024), p2_sdesc(ka + off, 16, 1024),
                     idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[x]);
      };
      // O_x (+)= P_x(j) V(j); P_x sits in the first 64 columns of S_x as packed bf16
      auto issue_pv = [&](int x, int j) {
        const int st = j & 1;
        const uint32_t va = smem_u32(s_v + st * P2_TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t db = p2_sdesc(va + uint32_t(kk) * 2048, P2_SUB_BYTES, 1024);
          tc_mma_f16_ts(tmem_base + 256u + uint32_t(x * 128), tmem_base + uint32_t(x * 128) + uint32_t(kk * 8), db,
                        idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&o_done[x]);
      };
      if (ok) ok = mbar_wait(&k_full[0], 0, p.status, ST_TIMEOUT_FULL);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        if (act_b) issue_s(1, 0);
        tc_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        const bool more = j + 1 < n_tiles;
        bool v_waited = false, k_waited = false;
        for (int x = 0; x < 2 && ok; ++x) {
          const int n_x = x == 0 ? n_a : n_b;
          if (j >= n_x) continue;
          ok = mbar_wait(&p_ready[x], uint32_t(j) & 1u, p.status, ST_TIMEOUT_FULL);
          if (ok && !v_waited) {
            ok = mbar_wait(&v_full[st], uint32_t(j >> 1) & 1u, p.status, ST_TIMEOUT_FULL);
            v_waited = true;
          }
          if (!ok) break;
          tc_fence_after();
          issue_pv(x, j);
          if (j + 1 < n_x) {
            if (!k_waited) {
              ok = mbar_wait(&k_full[st ^ 1], uint32_t((j + 1) >> 1) & 1u, p.status, ST_TIMEOUT_FULL);
              k_waited = true;
              if (!ok) break;
              tc_fence_after();
            }
            issue_s(x, j + 1);
          }
        }
        if (!ok) break;
        tc_commit(&v_empty[st]);
        if (more && k_waited) tc_commit(&k_empty[st ^ 1]);
      }
      if (!ok) *s_abort = 1;
    }
  } else {
    // ------------------------------------------------ softmax of one query tile (x = 0: A, 1: B)
    const int x = (warp - 2) >> 2;
    const int n_x = x == 0 ? n_a : n_b;
    const int kv_end_x = x == 0 ? kv_end_a : kv_end_b;
    const int lane_group = warp & 3;                         // TMEM lanes this warp may touch
    const int row = lane_group * 32 + lane;
    const uint32_t lane_addr = uint32_t(lane_group * 32) << 16;
    const uint32_t ts = tmem_base + lane_addr + uint32_t(x * 128);           // S_x, then P_x
    const uint32_t to = tmem_base + lane_addr + 256u + uint32_t(x * 128);    // O_x
    const int qrow = q0 + x * P2_BM + row;                   // row among the sequence's new tokens
    const int qpos = offset + qrow;                          // last key position this row may see
    float m_ref = 0.f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_x && ok; ++j) {
      if (*s_abort || !mbar_wait(&s_full[x], uint32_t(j) & 1u, p.status, ST_TIMEOUT_ACC_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(ts + uint32_t(c * 32), *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
      tmem_ld_wait();
      const int col0 = j * P2_BN;
      const bool need_mask = (col0 + P2_BN - 1 > offset + q0 + x * P2_BM) || (col0 + P2_BN > kv_end_x);
      if (need_mask) {
#pragma unroll
        for (int t = 0; t < 128; ++t) {
          const int col = col0 + t;
          if (col > qpos || col >= kv_end_x) s[t] = 0xff800000u;          // -inf
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int t = 0; t < 128; ++t) mx = fmaxf(mx, __uint_as_float(s[t]));
      mx *= p.scale_log2;
      if (j == 0) {
        m_ref = (mx == -INFINITY) ? 0.f : mx;
      } else if (__any_sync(__activemask(), mx > m_ref + P2_RESCALE_THRESHOLD)) {
        // some row of this warp outgrew its reference: bring O (complete up to tile j - 1) to the new one
        if (!mbar_wait(&o_done[x], uint32_t(j - 1) & 1u, p.status, ST_TIMEOUT_ACC_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const float m_new = fmaxf(m_ref, mx);
        const float f = exp2f(m_ref - m_new);
        m_ref = m_new;
        l *= f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(to + uint32_t(c * 32), r);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 32; ++t) r[t] = __float_as_uint(__uint_as_float(r[t]) * f);
          tmem_st_32x32(to + uint32_t(c * 32), r);
        }
        tmem_st_wait();
      }
      float rs = 0.f;
      uint32_t u[64];
#pragma unroll
      for (int t = 0; t < 64; ++t) {
        float e0, e1;
        const float a0 = fmaf(__uint_as_float(s[2 * t]), p.scale_log2, -m_ref);
        const float a1 = fmaf(__uint_as_float(s[2 * t + 1]), p.scale_log2, -m_ref);
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(a0));
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(a1));
        rs += e0 + e1;
        u[t] = pack_bf16(e0, e1);
      }
      tmem_st_32x32(ts, *reinterpret_cast<uint32_t(*)[32]>(&u[0]));
      tmem_st_32x32(ts + 32u, *reinterpret_cast<uint32_t(*)[32]>(&u[32]));
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_ready[x]);
      l += rs;
    }
    if (!ok) *s_abort = 1;
    if (ok && n_x > 0 && mbar_wait(&o_done[x], uint32_t(n_x - 1) & 1u, p.status, ST_TIMEOUT_ACC_FULL)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = p.out + ((long long)(q_begin + qrow) * p.Hq + h) * P2_D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(to + uint32_t(c * 32), r);
        tmem_ld_wait();
        if (qrow < q_len) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[q * 8 + 0]) * inv, __uint_as_float(r[q * 8 + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(r[q * 8 + 2]) * inv, __uint_as_float(r[q * 8 + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(r[q * 8 + 4]) * inv, __uint_as_float(r[q * 8 + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(r[q * 8 + 6]) * inv, __uint_as_float(r[q * 8 + 7]) * inv);
            reinterpret_cast<uint4*>(dst + c * 32)[q] = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

void launch_prefill_attention_tc2(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                                  const int* cu_seqlens_q, const int* kv_lens, void* out, long long total_q,
                                  int num_seqs, int max_q_len, int Hq, int Hkv, int block_size, int max_blocks,
                                  int num_blocks, float scale, uint32_t* status, cudaStream_t stream) {
  if (num_seqs == 0 || max_q_len == 0) return;
  if (Hq % Hkv != 0) throw std::runtime_error("prefill attention: Hq must be a multiple of Hkv");
  int box_rows = P2_BN;
  while (box_rows > block_size || block_size % box_rows != 0) box_rows >>= 1;
  if (box_rows < 8) throw std::runtime_error("prefill attention: block_size must be a multiple of 8");
  PrefillTc2Params p{};
  p.block_tables = block_tables;
  p.cu_q = cu_seqlens_q;
  p.kv_lens = kv_lens;
  p.out = reinterpret_cast<bf16*>(out);
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.block_size = block_size;
  p.box_rows = box_rows;
  p.max_blocks = max_blocks;
  p.num_blocks = num_blocks;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  const CUtensorMap tq = make_tmap_bf16_2d(q, (uint64_t)total_q, (uint64_t)Hq * P2_D, (uint64_t)Hq * P2_D, P2_BM, 64);
  const uint64_t rows = (uint64_t)num_blocks * Hkv * block_size;
  const CUtensorMap tk = make_tmap_bf16_2d(k_cache, rows, P2_D, P2_D, box_rows, 64);
  const CUtensorMap tv = make_tmap_bf16_2d(v_cache, rows, P2_D, P2_D, box_rows, 64);
  const int smem = 6 * P2_TILE_BYTES + 256 + 1024;
  cudaFuncSetAttribute(prefill_attn_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  dim3 grid((max_q_len + 2 * P2_BM - 1) / (2 * P2_BM), Hq, num_seqs);
  prefill_attn_tc2_kernel<<<grid, P2_THREADS, smem, stream>>>(tq, tk, tv, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("prefill attention (tcgen05, 2 tiles) launch: ") + cudaGetErrorString(e));
}

}  // namespace fc
