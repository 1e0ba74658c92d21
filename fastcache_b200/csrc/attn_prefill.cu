// Causal prefill attention over the paged pool.
//
// The K/V rows of the new tokens are already in the pool (the fused rotary/store
// op ran before), so this kernel reads every key and value through the block
// table.  That one path covers plain prefill, prefix-cache hits (queries are the
// last q_len rows of a longer kv_len) and chunked prefill.
//
// Grid (q tile of 64 rows, query head, request); heavy (late) q tiles are
// scheduled first.  4 warps x 16 query rows; K/V tiles of 64 rows, double-buffered
// with cp.async into XOR-swizzled shared memory; S = Q K^T and O += P V on
// mma.sync.m16n8k16 with the online-softmax recurrence in registers.
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

constexpr int PF_BM = 64;
constexpr int PF_BN = 64;
constexpr int PF_THREADS = 128;

template <int D>
__global__ void __launch_bounds__(PF_THREADS)
prefill_attn_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                    const int* __restrict__ block_tables, const int* __restrict__ cu_q,
                    const int* __restrict__ kv_lens, bf16* __restrict__ out, int Hq, int Hkv, int block_size,
                    int max_blocks, int num_blocks, float scale_log2, uint32_t* status) {
  constexpr int CH = D / 8;
  constexpr int Q_BYTES = PF_BM * D * 2;
  constexpr int T_BYTES = PF_BN * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t s_q = smem_u32(smem);
  const uint32_t s_kv = s_q + Q_BYTES;          // stage s: K at s * 2 * T_BYTES, V after it

  const int seq = blockIdx.z, h = blockIdx.y;
  const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
  const int q_tile = (gridDim.x - 1 - blockIdx.x);          // late tiles (most keys) first
  const int q0 = q_tile * PF_BM;
  if (q0 >= q_len) return;
  const int kv_len = kv_lens[seq];
  const int offset = kv_len - q_len;                        // query row i sits at kv position offset + i
  const int hk = h / (Hq / Hkv);
  const int* bt = block_tables + (long long)seq * max_blocks;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  const int kv_end = min(kv_len, offset + q0 + PF_BM);      // keys visible to this q tile
  const int n_tiles = (kv_end + PF_BN - 1) / PF_BN;

  // ---- Q tile -> smem
#pragma unroll
  for (int i = 0; i < (PF_BM * CH) / PF_THREADS; ++i) {
    const int c = threadIdx.x + i * PF_THREADS;
    const int r = c / CH, ch = c % CH;
    const bool valid = q0 + r < q_len;
    const bf16* src = q + ((long long)(q_begin + (valid ? q0 + r : 0)) * Hq + h) * D + ch * 8;
    cp_async16(s_q + swz<D>(r, ch), src, valid);
  }
  auto load_tile = [&](int tile, int stage) {
    const uint32_t sk = s_kv + stage * 2 * T_BYTES;
    const uint32_t sv = sk + T_BYTES;
    const int row0 = tile * PF_BN;
#pragma unroll
    for (int i = 0; i < (PF_BN * CH) / PF_THREADS; ++i) {
      const int c = threadIdx.x + i * PF_THREADS;
      const int r = c / CH, ch = c % CH;
      const int tok = row0 + r;
      bool valid = tok < kv_end;
      long long off = 0;
      if (valid) {
        const int blk = bt[tok / block_size];
        if (blk < 0 || blk >= num_blocks) {
          report(status, ST_BAD_INDEX);
          valid = false;
        } else {
          off = (((long long)blk * Hkv + hk) * block_size + tok % block_size) * D + ch * 8;
        }
      }
      cp_async16(sk + swz<D>(r, ch), k_cache + off, valid);
      cp_async16(sv + swz<D>(r, ch), v_cache + off, valid);
    }
  };
  load_tile(0, 0);
  cp_async_commit();                                         // group 0: Q + tile 0

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  uint32_t qa[D / 16][4];
  const int qrow0 = offset + q0 + warp * 16 + g;             // kv position of this thread's first row
  const int qrow1 = qrow0 + 8;

  for (int it = 0; it < n_tiles; ++it) {
    if (it + 1 < n_tiles) load_tile(it + 1, (it + 1) & 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const int mat = lane >> 3;
        const int r = warp * 16 + (mat & 1) * 8 + (lane & 7);
        const int ch = kk * 2 + (mat >> 1);
        ldsm_x4(s_q + swz<D>(r, ch), qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
      }
    }
    const uint32_t sk = s_kv + (it & 1) * 2 * T_BYTES;
    const uint32_t sv = sk + T_BYTES;

    float sc[PF_BN / 8][4];
#pragma unroll
    for (int n = 0; n < PF_BN / 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < PF_BN / 16; ++np) {
        const int mat = lane >> 3;
        const int r = np * 16 + (mat >> 1) * 8 + (lane & 7);
        const int ch = kk * 2 + (mat & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(sk + swz<D>(r, ch), b0, b1, b2, b3);
        mma_bf16(sc[2 * np], qa[kk], b0, b1);
        mma_bf16(sc[2 * np + 1], qa[kk], b2, b3);
      }
    }
    // ---- scale, causal mask (only tiles that touch the diagonal or the end), row max
    const int col0 = it * PF_BN;
    const bool need_mask = (col0 + PF_BN - 1 > offset + q0 + warp * 16) || (col0 + PF_BN > kv_end);
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < PF_BN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int col = col0 + n * 8 + 2 * t + e;
        float a = sc[n][e] * scale_log2, b = sc[n][2 + e] * scale_log2;
        if (need_mask) {
          if (col > qrow0 || col >= kv_end) a = -INFINITY;
          if (col > qrow1 || col >= kv_end) b = -INFINITY;
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
    const float cor0 = exp2f(m0 - base0), cor1 = exp2f(m1 - base1);
    m0 = nm0;
    m1 = nm1;
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int n = 0; n < PF_BN / 8; ++n) {
      sc[n][0] = exp2f(sc[n][0] - base0);
      sc[n][1] = exp2f(sc[n][1] - base0);
      sc[n][2] = exp2f(sc[n][2] - base1);
      sc[n][3] = exp2f(sc[n][3] - base1);
      rs0 += sc[n][0] + sc[n][1];
      rs1 += sc[n][2] + sc[n][3];
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
    for (int ks = 0; ks < PF_BN / 16; ++ks) {
      uint32_t pa[4];
      pa[0] = pack_bf16(sc[2 * ks][0], sc[2 * ks][1]);
      pa[1] = pack_bf16(sc[2 * ks][2], sc[2 * ks][3]);
      pa[2] = pack_bf16(sc[2 * ks + 1][0], sc[2 * ks + 1][1]);
      pa[3] = pack_bf16(sc[2 * ks + 1][2], sc[2 * ks + 1][3]);
#pragma unroll
      for (int jp = 0; jp < D / 16; ++jp) {
        const int mat = lane >> 3;
        const int r = ks * 16 + (mat & 1) * 8 + (lane & 7);
        const int ch = jp * 2 + (mat >> 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(sv + swz<D>(r, ch), b0, b1, b2, b3);
        mma_bf16(o[2 * jp], pa, b0, b1);
        mma_bf16(o[2 * jp + 1], pa, b2, b3);
      }
    }
    __syncthreads();                                         // stage (it & 1) may be overwritten next round
  }
  cp_async_wait<0>();

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    const int c = j * 8 + 2 * t;
    if (r0 < q_len)
      *reinterpret_cast<uint32_t*>(out + ((long long)(q_begin + r0) * Hq + h) * D + c) =
          pack_bf16(o[j][0] * inv0, o[j][1] * inv0);
    if (r1 < q_len)
      *reinterpret_cast<uint32_t*>(out + ((long long)(q_begin + r1) * Hq + h) * D + c) =
          pack_bf16(o[j][2] * inv1, o[j][3] * inv1);
  }
}

void launch_prefill_attention(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                              const int* cu_seqlens_q, const int* kv_lens, void* out, int num_seqs, int max_q_len,
                              int Hq, int Hkv, int D, int block_size, int max_blocks, int num_blocks, float scale,
                              uint32_t* status, cudaStream_t stream) {
  if (num_seqs == 0 || max_q_len == 0) return;
  if (Hq % Hkv != 0) throw std::runtime_error("prefill attention: Hq must be a multiple of Hkv");
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid((max_q_len + PF_BM - 1) / PF_BM, Hq, num_seqs);
  const int smem = PF_BM * D * 2 + 2 * 2 * PF_BN * D * 2;
  auto launch = [&](auto kern) {
    // set on every launch: both head-dim instantiations share this lambda's function-pointer type
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    kern<<<grid, PF_THREADS, smem, stream>>>((const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                                             block_tables, cu_seqlens_q, kv_lens, (bf16*)out, Hq, Hkv, block_size,
                                             max_blocks, num_blocks, scale_log2, status);
  };
  if (D == 128) launch(prefill_attn_kernel<128>);
  else if (D == 64) launch(prefill_attn_kernel<64>);
  else throw std::runtime_error("prefill attention: head_dim must be 64 or 128");
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("prefill attention launch: ") + cudaGetErrorString(e));
}

}  // namespace fc
