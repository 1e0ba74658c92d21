// Paged decode attention: one query row per request over its (possibly compressed) K/V in the pool.
//
// Grid (request, kv head, kv split).  A CTA streams 64-row K and V tiles of its
// kv head through a 3-stage cp.async ring (16-byte copies, XOR-swizzled rows,
// zero fill past the context), gathering rows through the block table.  The G =
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

#include "kernels.h"
#include "mma.cuh"
#include "ptx.cuh"

namespace fc {

using bf16 = __nv_bfloat16;

constexpr int DEC_TILE = 64;      // kv rows per stage
constexpr int DEC_STAGES = 3;
constexpr int DEC_THREADS = 128;

template <int D>
__global__ void __launch_bounds__(DEC_THREADS)
decode_attn_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                   const int* __restrict__ block_tables, const int* __restrict__ context_lens,
                   bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_lse, int Hq,
                   int Hkv, int block_size, int max_blocks, int num_blocks, int splits, float scale_log2,
                   uint32_t* status) {
  constexpr int CH = D / 8;                  // 16-byte chunks per row
  constexpr int TILE_BYTES = DEC_TILE * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t s_base = smem_u32(smem);
  // stage s: K tile at s * 2 * TILE_BYTES, V tile right after

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
      qa[kk][0] = (g < G) ? *reinterpret_cast<const uint32_t*>(q0 + g * D + c0) : 0u;
      qa[kk][1] = (g + 8 < G) ? *reinterpret_cast<const uint32_t*>(q0 + (g + 8) * D + c0) : 0u;
      qa[kk][2] = (g < G) ? *reinterpret_cast<const uint32_t*>(q0 + g * D + c0 + 8) : 0u;
      qa[kk][3] = (g + 8 < G) ? *reinterpret_cast<const uint32_t*>(q0 + (g + 8) * D + c0 + 8) : 0u;
    }
  }

  auto load_tile = [&](int tile, int stage) {
    const uint32_t sk = s_base + stage * 2 * TILE_BYTES;
    const uint32_t sv = sk + TILE_BYTES;
    const int row0 = tile * DEC_TILE;
#pragma unroll
    for (int i = 0; i < (DEC_TILE * CH) / DEC_THREADS; ++i) {
      const int c = threadIdx.x + i * DEC_THREADS;
      const int r = c / CH, ch = c % CH;
      const int tok = row0 + r;
      bool valid = tok < ctx;
      long long off = 0;
      if (valid) {
        const int blk = bt[tok / block_size];
        if (blk < 0 || blk >= num_blocks) {
          report(status, ST_BAD_INDEX);
          valid = false;
        } else {
          off = (((long long)blk * block_size + tok % block_size) * Hkv + hk) * D + ch * 8;
        }
      }
      cp_async16(sk + swz<D>(r, ch), k_cache + off, valid);
      cp_async16(sv + swz<D>(r, ch), v_cache + off, valid);
    }
  };

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

#pragma unroll
  for (int s = 0; s < DEC_STAGES - 1; ++s) {
    if (s < n_tiles) load_tile(tile0 + s, s);
    cp_async_commit();
  }

  for (int it = 0; it < n_tiles; ++it) {
    cp_async_wait<DEC_STAGES - 2>();
    __syncthreads();
    {   // prefetch tile it + STAGES - 1 into the stage that was consumed in the previous iteration
      const int nxt = it + DEC_STAGES - 1;
      if (nxt < n_tiles) load_tile(tile0 + nxt, nxt % DEC_STAGES);
      cp_async_commit();
    }
    const int stage = it % DEC_STAGES;
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
      ldsm_x4(sk + swz<D>(r, ch), b0, b1, b2, b3);
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
      ldsm_x4_t(sv + swz<D>(r, ch), b0, b1, b2, b3);
      mma_bf16(o[2 * jp], pa, b0, b1);
      mma_bf16(o[2 * jp + 1], pa, b2, b3);
    }
  }
  cp_async_wait<0>();
  __syncthreads();

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
}

// out[b, h, :] = sum_s w_s * part_o[b, h, s, :],  w_s = 2^(lse_s - max) / sum
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                    bf16* __restrict__ out, int splits, int D) {
  const long long bh = blockIdx.x;
  const float* lse = part_lse + bh * splits;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, lse[s]);
  float den = 0.f;
  for (int s = 0; s < splits; ++s) den += (lse[s] == -INFINITY) ? 0.f : exp2f(lse[s] - mx);
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float acc = 0.f;
    if (mx != -INFINITY) {
      for (int s = 0; s < splits; ++s) {
        const float w = (lse[s] == -INFINITY) ? 0.f : exp2f(lse[s] - mx);
        acc += w * part_o[(bh * splits + s) * D + c];
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
                             float scale, uint32_t* status, cudaStream_t stream) {
  if (B == 0) return;
  if (Hq % Hkv != 0 || Hq / Hkv > 16) throw std::runtime_error("decode attention: group size must divide and be <= 16");
  if (splits > 1 && (part_o == nullptr || part_lse == nullptr))
    throw std::runtime_error("decode attention: split-KV needs scratch");
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(B, Hkv, splits);
  const int smem = DEC_STAGES * 2 * DEC_TILE * D * 2;
  auto launch = [&](auto kern) {
    static bool configured = false;
    if (!configured) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      configured = true;
    }
    kern<<<grid, DEC_THREADS, smem, stream>>>((const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                                              block_tables, context_lens, (bf16*)out, part_o, part_lse, Hq, Hkv,
                                              block_size, max_blocks, num_blocks, splits, scale_log2, status);
  };
  if (D == 128) launch(decode_attn_kernel<128>);
  else if (D == 64) launch(decode_attn_kernel<64>);
  else throw std::runtime_error("decode attention: head_dim must be 64 or 128");
  if (splits > 1) decode_merge_kernel<<<B * Hq, 128, 0, stream>>>(part_o, part_lse, (bf16*)out, splits, D);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("decode attention launch: ") + cudaGetErrorString(e));
}

}  // namespace fc
