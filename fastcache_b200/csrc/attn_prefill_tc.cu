// Causal prefill attention on tcgen05 (head_dim 128), reading K/V through the block table.
//
// One CTA owns 128 query rows of one head and walks the visible keys in tiles of 128 rows:
//   warp 0      TMA: the Q tile once, then K and V tiles (boxes that never straddle a pool block)
//               into 2-stage rings, 128-byte swizzle
//   warp 1      tcgen05.mma issuer:  S = Q K^T  (M128 x N128, K = head_dim, both operands K-major,
//               accumulator in TMEM, two S buffers) and  O_tile = P V  (A = P from shared memory,
//               B = V as an MN-major operand straight from its [rows, D] tile, fresh accumulator)
//   warps 2-5   one query row per thread: tcgen05.ld of S, running max / sum in the exp2 domain,
//               P written to shared memory as bf16 in the swizzled K-major layout, then the tile's
//               O_tile is read from TMEM and folded into the row's register accumulator with the
//               rescale factor (the rescale never touches TMEM)
// S(j+1) is issued before P(j) V(j), so the tensor core computes the next scores while the softmax
// warps work on the current ones.
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

constexpr int PT_BM = 128;
constexpr int PT_BN = 128;
constexpr int PT_D = 128;
constexpr int PT_THREADS = 192;
constexpr int PT_TILE_BYTES = PT_BN * PT_D * 2;        // 32 KiB: two [128 x 64] sub-tiles
constexpr int PT_SUB_BYTES = PT_TILE_BYTES / 2;

// generic shared-memory matrix descriptor, 128-byte swizzle
__device__ __forceinline__ uint64_t pt_sdesc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((addr & 0x3FFFF) >> 4);
  d |= uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}

struct PrefillTcParams {
  const int* block_tables;
  const int* cu_q;
  const int* kv_lens;
  bf16* out;
  int Hq, Hkv, block_size, box_rows, max_blocks, num_blocks;
  float scale_log2;
  uint32_t* status;
};

__global__ void __launch_bounds__(PT_THREADS, 1)
prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const PrefillTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem;                                   // 32 KiB
  uint8_t* s_k = s_q + PT_TILE_BYTES;                    // 2 stages
  uint8_t* s_v = s_k + 2 * PT_TILE_BYTES;                // 2 stages
  uint8_t* s_p = s_v + 2 * PT_TILE_BYTES;                // 32 KiB
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_p + PT_TILE_BYTES);
  uint64_t* q_full = bars;            // [1]
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [2]
  uint64_t* s_free = bars + 11;       // [2] (128 arrivals)
  uint64_t* p_ready = bars + 13;      // [1] (128 arrivals)
  uint64_t* p_free = bars + 14;       // [1]
  uint64_t* o_full = bars + 15;       // [1]
  uint64_t* o_free = bars + 16;       // [1] (128 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.z, h = blockIdx.y;
  const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_begin;
  const int q0 = (gridDim.x - 1 - blockIdx.x) * PT_BM;        // late (long) tiles first
  if (q0 >= q_len) return;
  const int kv_len = p.kv_lens[seq];
  const int offset = kv_len - q_len;
  const int hk = h / (p.Hq / p.Hkv);
  const int kv_end = min(kv_len, offset + q0 + PT_BM);
  const int n_tiles = (kv_end + PT_BN - 1) / PT_BN;
  const int* bt = p.block_tables + (long long)seq * p.max_blocks;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&s_free[s], 128);
    }
    mbar_init(p_ready, 128);
    mbar_init(p_free, 1);
    mbar_init(o_full, 1);
    mbar_init(o_free, 128);
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  // V rows past the visible keys are never loaded; 0 * (uninitialised bits) must not produce NaN
  for (int i = threadIdx.x; i < 2 * PT_TILE_BYTES / 16; i += PT_THREADS)
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
  const uint32_t TM_S0 = tmem_base, TM_O = tmem_base + 256;   // S buffers at +0 / +128, O tile at +256

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA loader
    if (lane == 0) {
      mbar_expect_tx(q_full, PT_TILE_BYTES);
      tma_load_2d(s_q, &tm_q, q_full, h * PT_D, q_begin + q0);
      tma_load_2d(s_q + PT_SUB_BYTES, &tm_q, q_full, h * PT_D + 64, q_begin + q0);
      const int pieces = PT_BN / p.box_rows;
      for (int j = 0; j < n_tiles && !*s_abort; ++j) {
        const int st = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        const int row0 = j * PT_BN;
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
          uint8_t* dst = (which == 0 ? s_k : s_v) + st * PT_TILE_BYTES;
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
            tma_load_2d(dst + PT_SUB_BYTES + pc * p.box_rows * 128, tm, full, 64, grow);
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
      auto issue_s = [&](int j) {
        const int st = j & 1;
        const uint32_t use = uint32_t(j >> 1) & 1u;
        if (!mbar_wait(&k_full[st], use, p.status, ST_TIMEOUT_FULL)) return false;
        if (!mbar_wait(&s_free[st], use ^ 1u, p.status, ST_TIMEOUT_ACC_EMPTY)) return false;
        tc_fence_after();
        const uint32_t qa = smem_u32(s_q), ka = smem_u32(s_k + st * PT_TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = uint32_t(kk >> 2) * PT_SUB_BYTES + uint32_t(kk & 3) * 32;
          tc_mma_f16(TM_S0 + uint32_t(st * 128), pt_sdesc(qa + off, 16, 1024), pt_sdesc(ka + off, 16, 1024),
                     idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[st]);
        tc_commit(&k_empty[st]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        const int st = j & 1;
        ok = mbar_wait(p_ready, uint32_t(j) & 1u, p.status, ST_TIMEOUT_FULL) &&
             mbar_wait(&v_full[st], uint32_t(j >> 1) & 1u, p.status, ST_TIMEOUT_FULL) &&
             mbar_wait(o_free, (uint32_t(j) & 1u) ^ 1u, p.status, ST_TIMEOUT_ACC_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t pa = smem_u32(s_p), va = smem_u32(s_v + st * PT_TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // A = P: K-major, k-step of 16 kv rows = 32 bytes inside the 128-byte row of sub-tile kk / 4
          const uint64_t da = pt_sdesc(pa + uint32_t(kk >> 2) * PT_SUB_BYTES + uint32_t(kk & 3) * 32, 16, 1024);
          // B = V: MN-major ([kv rows, D] tile): 16 kv rows = 2048 bytes; the two 64-wide halves of D are
          // PT_SUB_BYTES apart (leading byte offset), groups of 8 kv rows 1024 bytes apart (stride)
          const uint64_t db = pt_sdesc(va + uint32_t(kk) * 2048, PT_SUB_BYTES, 1024);
          tc_mma_f16(TM_O, da, db, idesc_o, kk > 0 ? 1u : 0u);
        }
        tc_commit(o_full);
        tc_commit(&v_empty[st]);
        tc_commit(p_free);
      }
      if (!ok) *s_abort = 1;
    }
  } else {
    // ------------------------------------------------------- softmax + output accumulation
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;
    const uint32_t lane_addr = uint32_t(lane_group * 32) << 16;
    const int qpos = offset + q0 + row;                     // kv position this query row may see up to
    float m = -INFINITY, l = 0.f;
    float o[PT_D];
#pragma unroll
    for (int i = 0; i < PT_D; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j & 1;
      if (*s_abort || !mbar_wait(&s_full[st], uint32_t(j >> 1) & 1u, p.status, ST_TIMEOUT_ACC_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t ts = TM_S0 + uint32_t(st * 128) + lane_addr;
      const int col0 = j * PT_BN;
      const bool need_mask = (col0 + PT_BN - 1 > offset + q0) || (col0 + PT_BN > kv_end);
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(ts + uint32_t(c * 32), r);
        tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          float v = __uint_as_float(r[t]);
          if (need_mask) {
            const int col = col0 + c * 32 + t;
            if (col > qpos || col >= kv_end) v = -INFINITY;
          }
          mx = fmaxf(mx, v);
        }
      }
      const float m_new = fmaxf(m, mx * p.scale_log2);
      const float base = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = exp2f(m - base);
      m = m_new;
      // pass 2: probabilities -> shared memory (bf16, swizzled K-major), row sum
      if (!mbar_wait(p_free, (uint32_t(j) & 1u) ^ 1u, p.status, ST_TIMEOUT_EMPTY)) {
        ok = false;
        break;
      }
      float rs = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(ts + uint32_t(c * 32), r);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t u[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float pv[2];
#pragma unroll
            for (int z = 0; z < 2; ++z) {
              const int t = q * 8 + e * 2 + z;
              float v = __uint_as_float(r[t]) * p.scale_log2 - base;
              if (need_mask) {
                const int col = col0 + c * 32 + t;
                if (col > qpos || col >= kv_end) v = -INFINITY;
              }
              pv[z] = exp2f(v);
              rs += pv[z];
            }
            u[e] = pack_bf16(pv[0], pv[1]);
          }
          const int chunk = c * 4 + q;
          uint8_t* dst = s_p + (chunk >> 3) * PT_SUB_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(dst) = make_uint4(u[0], u[1], u[2], u[3]);
        }
      }
      tc_fence_before();
      mbar_arrive(&s_free[st]);
      fence_proxy_async();
      mbar_arrive(p_ready);
      l = l * corr + rs;
      // fold the tile's P V into the register accumulator
      if (!mbar_wait(o_full, uint32_t(j) & 1u, p.status, ST_TIMEOUT_ACC_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(TM_O + lane_addr + uint32_t(c * 32), r);
        tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 32; ++t) o[c * 32 + t] = o[c * 32 + t] * corr + __uint_as_float(r[t]);
      }
      tc_fence_before();
      mbar_arrive(o_free);
    }
    if (!ok) *s_abort = 1;
    if (ok && q0 + row < q_len) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = p.out + ((long long)(q_begin + q0 + row) * p.Hq + h) * PT_D;
#pragma unroll
      for (int c = 0; c < PT_D / 8; ++c) {
        uint4 u;
        u.x = pack_bf16(o[c * 8 + 0] * inv, o[c * 8 + 1] * inv);
        u.y = pack_bf16(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv);
        u.z = pack_bf16(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv);
        u.w = pack_bf16(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv);
        reinterpret_cast<uint4*>(dst)[c] = u;
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

bool prefill_attention_tc_supported(int D, int block_size) { return D == PT_D && block_size % 8 == 0; }

void launch_prefill_attention_tc(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                                 const int* cu_seqlens_q, const int* kv_lens, void* out, long long total_q,
                                 int num_seqs, int max_q_len, int Hq, int Hkv, int block_size, int max_blocks,
                                 int num_blocks, float scale, uint32_t* status, cudaStream_t stream) {
  if (num_seqs == 0 || max_q_len == 0) return;
  if (Hq % Hkv != 0) throw std::runtime_error("prefill attention: Hq must be a multiple of Hkv");
  int box_rows = PT_BN;
  while (box_rows > block_size || block_size % box_rows != 0) box_rows >>= 1;
  if (box_rows < 8) throw std::runtime_error("prefill attention: block_size must be a multiple of 8");
  PrefillTcParams p{};
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
  const CUtensorMap tq = make_tmap_bf16_2d(q, (uint64_t)total_q, (uint64_t)Hq * PT_D, (uint64_t)Hq * PT_D, PT_BM, 64);
  const uint64_t rows = (uint64_t)num_blocks * Hkv * block_size;
  const CUtensorMap tk = make_tmap_bf16_2d(k_cache, rows, PT_D, PT_D, box_rows, 64);
  const CUtensorMap tv = make_tmap_bf16_2d(v_cache, rows, PT_D, PT_D, box_rows, 64);
  const int smem = 6 * PT_TILE_BYTES + 256 + 1024;
  cudaFuncSetAttribute(prefill_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  dim3 grid((max_q_len + PT_BM - 1) / PT_BM, Hq, num_seqs);
  prefill_attn_tc_kernel<<<grid, PT_THREADS, smem, stream>>>(tq, tk, tv, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("prefill attention (tcgen05) launch: ") + cudaGetErrorString(e));
}

}  // namespace fc
