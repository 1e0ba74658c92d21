// Paged decode attention: one query row per request over its (possibly compressed) K/V in the pool.
//
// Grid (request, kv head, kv split).  A CTA streams 64-row K and V tiles of its
// kv head through a 3-stage ring filled by TMA (cp.async.bulk.tensor 2-D boxes with
// the 128-byte swizzle, completion on an mbarrier): the pool is head-major inside a
// block, so the rows of one head are a dense [rows, D] matrix and one elected thread
// moves a whole tile with a handful of instructions.  Boxes never straddle a pool
// block (box rows = min(64, block_size)); boxes wholly past the context are skipped
// and rows past it are masked.  The G =
// Hq / Hkv query heads that share the kv head form the 16-row A operand of
// mma.sync.m16n8k16 (rows >= G are zero); each of the 4 warps owns 16 of the 64
// rows of a tile and keeps its own running (max, sum, O[16 x D]).  The warps are
// merged through shared memory at the end.  With more than one split the CTA
// writes a normalised partial and its log-sum-exp to scratch and a second kernel
// merges the splits.
//
// This op is bound by HBM bandwidth (K and V are read exactly once, ~16 FLOP per
// byte), so the legacy tensor path is enough to keep the memory system busy; the
// tcgen05 path is used where the work is compute-bound.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <stdexcept>
#include <string>

#include "gemm.h"
#include "kernels.h"
#include "launch.h"
#include "mma.cuh"
#include "ptx.cuh"

namespace fc {

using bf16 = __nv_bfloat16;

constexpr int DEC_TILE = 64;      // kv rows per stage
constexpr int DEC_STAGES = 3;
constexpr int DEC_THREADS = 128;

// byte offset of 16-byte chunk `chunk` of row `row` inside a TMA-swizzled tile:
// sub-tiles of [64 rows x 128 bytes], chunk index XOR (row mod 8) inside the 128-byte row
__device__ __forceinline__ uint32_t tswz(int row, int chunk) {
  return uint32_t((chunk >> 3) * (DEC_TILE * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// Split-KV without a second kernel: every CTA of a (request, KV head) counts itself in after its partial results are
// written; the last one to arrive merges all splits of the group's query heads
//     out[b, h, :] = sum_s w_s * part_o[b, h, s, :],  w_s = 2^(lse_s - max) / sum
// and puts the counter back to zero for the next launch (also a replay from a CUDA graph).
template <int D>
__device__ __forceinline__ void decode_merge_last(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                                  bf16* __restrict__ out, int* __restrict__ counters, int b, int hk,
                                                  int G, int Hq, int Hkv, int splits) {
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(counters + b * Hkv + hk, 1);
    s_last = old == splits - 1 ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < G * D; idx += DEC_THREADS) {
    const int r = idx / D, c = idx - r * D;
    const long long bh = (long long)b * Hq + hk * G + r;
    const float* lse = part_lse + bh * splits;
    float mx = -INFINITY;
    for (int s = 0; s < splits; ++s) mx = fmaxf(mx, __ldcg(lse + s));
    float acc = 0.f, den = 0.f;
    if (mx != -INFINITY) {
      for (int s = 0; s < splits; ++s) {
        const float l = __ldcg(lse + s);
        const float w = (l == -INFINITY) ? 0.f : exp2f(l - mx);
        den += w;
        acc += w * __ldcg(part_o + (bh * splits + s) * D + c);
      }
      acc /= den;
    }
    out[bh * D + c] = __float2bfloat16(acc);
  }
  if (threadIdx.x == 0) counters[b * Hkv + hk] = 0;
}

template <int D>
__global__ void __launch_bounds__(DEC_THREADS)
decode_attn_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const bf16* __restrict__ q, int box_rows, const int* __restrict__ block_tables, const int* __restrict__ context_lens,
                   bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_lse, int Hq,
                   int Hkv, int block_size, int max_blocks, int num_blocks, int splits, float scale_log2,
                   uint32_t* status, int* __restrict__ merge_counters) {
  constexpr int CH = D / 8;                  // 16-byte chunks per row
  constexpr int TILE_BYTES = DEC_TILE * D * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_u32(smem);
  // stage s: K tile at s * 2 * TILE_BYTES, V tile right after; a tile is D/64 sub-tiles of [64 rows x 128 B]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + DEC_STAGES * 2 * TILE_BYTES);
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < DEC_STAGES; ++s) mbar_init(&full_bar[s], 1);
    fence_barrier_init();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  __syncthreads();
  pdl_wait();                                // q and the new K/V rows come from the kernels before this one
  // the rows were written with ordinary stores and are read by TMA: order the two proxies
  asm volatile("fence.proxy.async.global;" ::: "memory");

  const int b = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int G = Hq / Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  const int ctx = context_lens[b];
  const int tiles_total = (ctx + DEC_TILE - 1) / DEC_TILE;
  const int tiles_per = (tiles_total + splits - 1) / splits;
  const int tile0 = split * tiles_per;
  const int tile1 = min(tiles_total, tile0 + tiles_per);
  const int n_tiles = max(0, tile1 - tile0);
  const int* bt = block_tables + (long long)b * max_blocks;

  // ---- Q fragments (A operand): rows = heads of this group, zero beyond G
  uint32_t qa[D / 16][4];
  {
    const bf16* q0 = q + ((long long)b * Hq + (long long)hk * G) * D;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const int c0 = kk * 16 + 2 * t;
      // q was written by the kernel before this one while this grid may already have been resident
      // (programmatic dependent launch): read it through L2, never through the read-only path
      qa[kk][0] = (g < G) ? __ldcg(reinterpret_cast<const uint32_t*>(q0 + g * D + c0)) : 0u;
      qa[kk][1] = (g + 8 < G) ? __ldcg(reinterpret_cast<const uint32_t*>(q0 + (g + 8) * D + c0)) : 0u;
      qa[kk][2] = (g < G) ? __ldcg(reinterpret_cast<const uint32_t*>(q0 + g * D + c0 + 8)) : 0u;
      qa[kk][3] = (g + 8 < G) ? __ldcg(reinterpret_cast<const uint32_t*>(q0 + (g + 8) * D + c0 + 8)) : 0u;
    }
  }

  // one thread: TMA boxes of tile `tile` into `stage`
  auto load_tile = [&](int tile, int stage) {
    uint8_t* sk = smem + stage * 2 * TILE_BYTES;
    uint8_t* sv = sk + TILE_BYTES;
    const int row0 = tile * DEC_TILE;
    const int pieces = DEC_TILE / box_rows;
    constexpr int SUBS = D / 64;
    uint32_t bytes = 0;
    for (int pc = 0; pc < pieces; ++pc)
      if (row0 + pc * box_rows < ctx) bytes += uint32_t(2 * SUBS * box_rows * 128);
    mbar_expect_tx(&full_bar[stage], bytes);
    for (int pc = 0; pc < pieces; ++pc) {
      const int tok = row0 + pc * box_rows;
      if (tok >= ctx) break;
      int blk = bt[tok / block_size];
      if (blk < 0 || blk >= num_blocks) {
        report(status, ST_BAD_INDEX);
        blk = 0;                          // keep the byte count consistent; the rows are garbage either way
      }
      const int grow = (blk * Hkv + hk) * block_size + tok % block_size;
#pragma unroll
      for (int sub = 0; sub < SUBS; ++sub) {
        const int soff = sub * (DEC_TILE * 128) + pc * box_rows * 128;
        tma_load_2d(sk + soff, &tm_k, &full_bar[stage], sub * 64, grow);
        tma_load_2d(sv + soff, &tm_v, &full_bar[stage], sub * 64, grow);
      }
    }
  };

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  if (n_tiles <= DEC_STAGES) {
    // Boxes past the context are never loaded.  In a short run their shared memory has not been
    // written at all, and 0 * (uninitialised V) could be NaN, so clear the V tiles once.
    for (int s = 0; s < n_tiles; ++s) {
      uint4* v = reinterpret_cast<uint4*>(smem + s * 2 * TILE_BYTES + TILE_BYTES);
      for (int i = threadIdx.x; i < TILE_BYTES / 16; i += DEC_THREADS) v[i] = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async();
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < DEC_STAGES; ++s)
      if (s < n_tiles) load_tile(tile0 + s, s);
  }
  bool alive = true;
  for (int it = 0; it < n_tiles; ++it) {
    const int stage = it % DEC_STAGES;
    if (!mbar_wait(&full_bar[stage], (it / DEC_STAGES) & 1, status, ST_TIMEOUT_FULL)) {
      alive = false;
      break;
    }
    const uint32_t sk = s_base + stage * 2 * TILE_BYTES;
    const uint32_t sv = sk + TILE_BYTES;
    const int wrow = warp * 16;                         // this warp's 16 rows of the tile
    const int tok_base = (tile0 + it) * DEC_TILE + wrow;

    // ---- S = Q K^T for 16 kv rows: two n8 tiles
    float sc[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const int mat = lane >> 3;
      const int r = wrow + (mat >> 1) * 8 + (lane & 7);
      const int ch = kk * 2 + (mat & 1);
      uint32_t b0, b1, b2, b3;
      ldsm_x4(sk + tswz(r, ch), b0, b1, b2, b3);
      mma_bf16(sc[0], qa[kk], b0, b1);
      mma_bf16(sc[1], qa[kk], b2, b3);
    }
    // ---- mask rows past the context, online softmax (rows g and g + 8 of the group)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int tok = tok_base + n * 8 + 2 * t + e;
        if (tok >= ctx) {
          sc[n][e] = -INFINITY;
          sc[n][2 + e] = -INFINITY;
        } else {
          sc[n][e] *= scale_log2;
          sc[n][2 + e] *= scale_log2;
        }
        mx0 = fmaxf(mx0, sc[n][e]);
        mx1 = fmaxf(mx1, sc[n][2 + e]);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
    const float base0 = (nm0 == -INFINITY) ? 0.f : nm0, base1 = (nm1 == -INFINITY) ? 0.f : nm1;
    const float cor0 = exp2f(m0 - base0), cor1 = exp2f(m1 - base1);
    m0 = nm0;
    m1 = nm1;
    float rs0 = 0.f, rs1 = 0.f;
    uint32_t pa[4];
    {
      float p[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        p[n][0] = exp2f(sc[n][0] - base0);
        p[n][1] = exp2f(sc[n][1] - base0);
        p[n][2] = exp2f(sc[n][2] - base1);
        p[n][3] = exp2f(sc[n][3] - base1);
        rs0 += p[n][0] + p[n][1];
        rs1 += p[n][2] + p[n][3];
      }
      pa[0] = pack_bf16(p[0][0], p[0][1]);
      pa[1] = pack_bf16(p[0][2], p[0][3]);
      pa[2] = pack_bf16(p[1][0], p[1][1]);
      pa[3] = pack_bf16(p[1][2], p[1][3]);
    }
    l0 = l0 * cor0 + rs0;
    l1 = l1 * cor1 + rs1;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      o[j][0] *= cor0;
      o[j][1] *= cor0;
      o[j][2] *= cor1;
      o[j][3] *= cor1;
    }
    // ---- O += P V
#pragma unroll
    for (int jp = 0; jp < D / 16; ++jp) {
      const int mat = lane >> 3;
      const int r = wrow + (mat & 1) * 8 + (lane & 7);
      const int ch = jp * 2 + (mat >> 1);
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(sv + tswz(r, ch), b0, b1, b2, b3);
      mma_bf16(o[2 * jp], pa, b0, b1);
      mma_bf16(o[2 * jp + 1], pa, b2, b3);
    }
    __syncthreads();                       // every warp is done with this stage
    if (threadIdx.x == 0 && it + DEC_STAGES < n_tiles) load_tile(tile0 + it + DEC_STAGES, stage);
  }
  if (__syncthreads_or(!alive)) {
    // a TMA never landed: the status word is set.  The split's cells are still written (weight zero), so the
    // merge kernel never mixes in what an earlier call left in the scratch
    for (int idx = threadIdx.x; idx < G * D; idx += DEC_THREADS) {
      const int r = idx / D, c = idx - r * D;
      const int hq = hk * G + r;
      if (splits == 1) {
        out[((long long)b * Hq + hq) * D + c] = __float2bfloat16(0.f);
      } else {
        part_o[(((long long)b * Hq + hq) * splits + split) * D + c] = 0.f;
        if (c == 0) part_lse[((long long)b * Hq + hq) * splits + split] = -INFINITY;
      }
    }
    if (splits > 1 && merge_counters != nullptr) decode_merge_last<D>(part_o, part_lse, out, merge_counters, b, hk, G, Hq, Hkv, splits);
    return;
  }

  // ---- merge the four warps (each saw a different quarter of every tile)
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  float* s_o = reinterpret_cast<float*>(smem);                 // [4][16][D]
  float* s_m = s_o + 4 * 16 * D;                               // [4][16]
  float* s_l = s_m + 64;                                       // [4][16]
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    const int c = j * 8 + 2 * t;
    float* r0 = s_o + (warp * 16 + g) * D + c;
    float* r1 = s_o + (warp * 16 + g + 8) * D + c;
    r0[0] = o[j][0];
    r0[1] = o[j][1];
    r1[0] = o[j][2];
    r1[1] = o[j][3];
  }
  if (t == 0) {
    s_m[warp * 16 + g] = m0;
    s_m[warp * 16 + g + 8] = m1;
    s_l[warp * 16 + g] = l0;
    s_l[warp * 16 + g + 8] = l1;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += DEC_THREADS) {
    const int r = idx / D, c = idx - r * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, s_m[w * 16 + r]);
    float acc = 0.f, ll = 0.f;
    if (mm != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = exp2f(s_m[w * 16 + r] - mm);
        acc += f * s_o[(w * 16 + r) * D + c];
        ll += f * s_l[w * 16 + r];
      }
    }
    const int hq = hk * G + r;
    const float val = (ll > 0.f) ? acc / ll : 0.f;
    if (splits == 1) {
      out[((long long)b * Hq + hq) * D + c] = __float2bfloat16(val);
    } else {
      part_o[(((long long)b * Hq + hq) * splits + split) * D + c] = val;
      if (c == 0)
        part_lse[((long long)b * Hq + hq) * splits + split] = (ll > 0.f) ? (mm + log2f(ll)) : -INFINITY;
    }
  }
  if (splits > 1 && merge_counters != nullptr) decode_merge_last<D>(part_o, part_lse, out, merge_counters, b, hk, G, Hq, Hkv, splits);
}

// out[b, h, :] = sum_s w_s * part_o[b, h, s, :],  w_s = 2^(lse_s - max) / sum
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                    bf16* __restrict__ out, int splits, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const long long bh = blockIdx.x;
  const float* lse = part_lse + bh * splits;
  // the partials come from the kernel right before this one: L2 loads, not the read-only path (see above)
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, __ldcg(lse + s));
  float den = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float l = __ldcg(lse + s);
    den += (l == -INFINITY) ? 0.f : exp2f(l - mx);
  }
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float acc = 0.f;
    if (mx != -INFINITY) {
      for (int s = 0; s < splits; ++s) {
        const float l = __ldcg(lse + s);
        const float w = (l == -INFINITY) ? 0.f : exp2f(l - mx);
        acc += w * __ldcg(part_o + (bh * splits + s) * D + c);
      }
      acc /= den;
    }
    out[bh * D + c] = __float2bfloat16(acc);
  }
}

int decode_attn_pick_splits(int B, int Hkv, int max_ctx, int num_sms) {
  const int ctas = B * Hkv;
  const int target = 2 * num_sms;
  if (ctas >= target) return 1;
  const int max_by_len = std::max(1, max_ctx / (4 * DEC_TILE));
  return std::max(1, std::min({(target + ctas - 1) / ctas, max_by_len, DECODE_MAX_SPLITS}));
}

void launch_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                             const int* context_lens, void* out, float* part_o, float* part_lse, int B, int Hq,
                             int Hkv, int D, int block_size, int max_blocks, int num_blocks, int splits,
                             float scale, uint32_t* status, cudaStream_t stream, int* merge_counters) {
  if (B == 0) return;
  if (Hq % Hkv != 0 || Hq / Hkv > 16) throw std::runtime_error("decode attention: group size must divide and be <= 16");
  if (splits > 1 && (part_o == nullptr || part_lse == nullptr))
    throw std::runtime_error("decode attention: split-KV needs scratch");
  int box_rows = DEC_TILE;
  while (box_rows > block_size || block_size % box_rows != 0) box_rows >>= 1;
  if (box_rows < 8) throw std::runtime_error("decode attention: block_size must be a multiple of 8");
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(B, Hkv, splits);
  const int smem = DEC_STAGES * 2 * DEC_TILE * D * 2 + 64 + 1024;
  const uint64_t rows = (uint64_t)num_blocks * Hkv * block_size;
  const CUtensorMap tk = make_tmap_bf16_2d(k_cache, rows, D, D, box_rows, 64);
  const CUtensorMap tv = make_tmap_bf16_2d(v_cache, rows, D, D, box_rows, 64);
  auto launch = [&](auto kern) {
    // set on every launch: both head-dim instantiations share this lambda's function-pointer type
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    launch_pdl(PDL_DECODE_ATTN, kern, grid, dim3(DEC_THREADS), smem, stream, tk, tv, (const bf16*)q, box_rows, block_tables,
               context_lens, (bf16*)out, part_o, part_lse, Hq, Hkv, block_size, max_blocks, num_blocks, splits,
               scale_log2, status, merge_counters);
  };
  if (D == 128) launch(decode_attn_kernel<128>);
  else if (D == 64) launch(decode_attn_kernel<64>);
  else throw std::runtime_error("decode attention: head_dim must be 64 or 128");
  // `merge_counters` (zero between launches, B * Hkv words): the last split of a (request, KV head) merges in the
  // attention kernel itself; without them a second kernel does
  if (splits > 1 && merge_counters == nullptr)
    launch_pdl(PDL_DECODE_MERGE, decode_merge_kernel, dim3(B * Hq), dim3(128), 0, stream, (const float*)part_o, (const float*)part_lse,
               (bf16*)out, splits, D);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("decode attention launch: ") + cudaGetErrorString(e));
}

}  // namespace fc
