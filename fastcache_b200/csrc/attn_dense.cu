// Non-causal attention for the vision towers (CLIP ViT-L: 577 tokens, 16 heads of 64;
// SigLIP: up to 1024 patches, 16 heads of 72; perceiver resampler: 64 queries over the
// patches, heads of 128).  Flash-style: the score matrix is never written to memory.
//
// q [B, Sq, H, D], k / v [B, Sk, H, D] with arbitrary batch / row / head strides (D contiguous),
// so the packed QKV output of one GEMM is consumed in place.  Head dims that are not a
// multiple of 16 (72) are zero-padded to the next multiple inside shared memory.  Optional
// key mask [B, Sk] (1 = attend) for ragged slices.
//
// Grid (q tile of 64 rows, head, batch); 4 warps x 16 rows; K/V tiles of 64 rows, double
// buffered with cp.async; rows padded by 16 bytes in shared memory (conflict-free ldmatrix);
// mma.sync m16n8k16 with the online-softmax recurrence in registers.
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

constexpr int DA_BM = 64;
constexpr int DA_BN = 64;
constexpr int DA_THREADS = 128;

struct DenseAttnParams {
  const bf16 *q, *k, *v;
  bf16* out;
  const uint8_t* key_mask;       // [B, Sk] or nullptr
  long long q_sb, q_ss, q_sh;    // element strides: batch, row, head
  long long k_sb, k_ss, k_sh;
  long long v_sb, v_ss, v_sh;
  int Sq, Sk, H, D;
  float scale_log2;
};

template <int DP>   // head dim padded to a multiple of 16
__global__ void __launch_bounds__(DA_THREADS) dense_attn_kernel(const DenseAttnParams p) {
  constexpr int PITCH = DP * 2 + 16;                 // bytes per shared-memory row
  constexpr int CH = DP / 8;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t s_q = smem_u32(smem);
  const uint32_t s_kv = s_q + DA_BM * PITCH;         // stage s: K at s * 2 * DA_BN * PITCH, V after it
  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * DA_BM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int valid_ch = p.D / 8;                      // D is a multiple of 8
  const int n_tiles = (p.Sk + DA_BN - 1) / DA_BN;

  const bf16* qb = p.q + b * p.q_sb + h * p.q_sh;
  const bf16* kb = p.k + b * p.k_sb + h * p.k_sh;
  const bf16* vb = p.v + b * p.v_sb + h * p.v_sh;

  for (int c = threadIdx.x; c < DA_BM * CH; c += DA_THREADS) {
    const int r = c / CH, ch = c % CH;
    const bool ok = (q0 + r < p.Sq) && ch < valid_ch;
    cp_async16(s_q + r * PITCH + ch * 16, qb + (ok ? (long long)(q0 + r) * p.q_ss + ch * 8 : 0), ok);
  }
  auto load_tile = [&](int tile, int stage) {
    const uint32_t sk = s_kv + stage * 2 * DA_BN * PITCH;
    const uint32_t sv = sk + DA_BN * PITCH;
    for (int c = threadIdx.x; c < DA_BN * CH; c += DA_THREADS) {
      const int r = c / CH, ch = c % CH;
      const int tok = tile * DA_BN + r;
      const bool ok = tok < p.Sk && ch < valid_ch;
      cp_async16(sk + r * PITCH + ch * 16, kb + (ok ? (long long)tok * p.k_ss + ch * 8 : 0), ok);
      cp_async16(sv + r * PITCH + ch * 16, vb + (ok ? (long long)tok * p.v_ss + ch * 8 : 0), ok);
    }
  };
  load_tile(0, 0);
  cp_async_commit();

  float o[DP / 8][4];
#pragma unroll
  for (int j = 0; j < DP / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  uint32_t qa[DP / 16][4];
  const uint8_t* mask = p.key_mask != nullptr ? p.key_mask + (long long)b * p.Sk : nullptr;

  for (int it = 0; it < n_tiles; ++it) {
    if (it + 1 < n_tiles) load_tile(it + 1, (it + 1) & 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int kk = 0; kk < DP / 16; ++kk) {
        const int mat = lane >> 3;
        const int r = warp * 16 + (mat & 1) * 8 + (lane & 7);
        const int ch = kk * 2 + (mat >> 1);
        ldsm_x4(s_q + r * PITCH + ch * 16, qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
      }
    }
    const uint32_t sk = s_kv + (it & 1) * 2 * DA_BN * PITCH;
    const uint32_t sv = sk + DA_BN * PITCH;
    float sc[DA_BN / 8][4];
#pragma unroll
    for (int n = 0; n < DA_BN / 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DP / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < DA_BN / 16; ++np) {
        const int mat = lane >> 3;
        const int r = np * 16 + (mat >> 1) * 8 + (lane & 7);
        const int ch = kk * 2 + (mat & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(sk + r * PITCH + ch * 16, b0, b1, b2, b3);
        mma_bf16(sc[2 * np], qa[kk], b0, b1);
        mma_bf16(sc[2 * np + 1], qa[kk], b2, b3);
      }
    }
    const int col0 = it * DA_BN;
    const bool need_mask = (col0 + DA_BN > p.Sk) || mask != nullptr;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < DA_BN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int col = col0 + n * 8 + 2 * t + e;
        float a = sc[n][e] * p.scale_log2, bb = sc[n][2 + e] * p.scale_log2;
        if (need_mask) {
          const bool dead = col >= p.Sk || (mask != nullptr && mask[col] == 0);
          if (dead) a = bb = -INFINITY;
        }
        sc[n][e] = a;
        sc[n][2 + e] = bb;
        mx0 = fmaxf(mx0, a);
        mx1 = fmaxf(mx1, bb);
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
    for (int n = 0; n < DA_BN / 8; ++n) {
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
    for (int j = 0; j < DP / 8; ++j) {
      o[j][0] *= cor0;
      o[j][1] *= cor0;
      o[j][2] *= cor1;
      o[j][3] *= cor1;
    }
#pragma unroll
    for (int ks = 0; ks < DA_BN / 16; ++ks) {
      uint32_t pa[4];
      pa[0] = pack_bf16(sc[2 * ks][0], sc[2 * ks][1]);
      pa[1] = pack_bf16(sc[2 * ks][2], sc[2 * ks][3]);
      pa[2] = pack_bf16(sc[2 * ks + 1][0], sc[2 * ks + 1][1]);
      pa[3] = pack_bf16(sc[2 * ks + 1][2], sc[2 * ks + 1][3]);
#pragma unroll
      for (int jp = 0; jp < DP / 16; ++jp) {
        const int mat = lane >> 3;
        const int r = ks * 16 + (mat & 1) * 8 + (lane & 7);
        const int ch = jp * 2 + (mat >> 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(sv + r * PITCH + ch * 16, b0, b1, b2, b3);
        mma_bf16(o[2 * jp], pa, b0, b1);
        mma_bf16(o[2 * jp + 1], pa, b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;
  bf16* ob = p.out + ((long long)b * p.Sq * p.H + h) * p.D;
#pragma unroll
  for (int j = 0; j < DP / 8; ++j) {
    const int c = j * 8 + 2 * t;
    if (c < p.D) {
      if (r0 < p.Sq)
        *reinterpret_cast<uint32_t*>(ob + (long long)r0 * p.H * p.D + c) = pack_bf16(o[j][0] * inv0, o[j][1] * inv0);
      if (r1 < p.Sq)
        *reinterpret_cast<uint32_t*>(ob + (long long)r1 * p.H * p.D + c) = pack_bf16(o[j][2] * inv1, o[j][3] * inv1);
    }
  }
}

void launch_dense_attention(const void* q, const void* k, const void* v, void* out, const uint8_t* key_mask,
                            int B, int Sq, int Sk, int H, int D, const long long* q_strides,
                            const long long* k_strides, const long long* v_strides, float scale,
                            cudaStream_t stream) {
  if (B == 0 || Sq == 0) return;
  if (D % 8 != 0 || D > 128) throw std::runtime_error("dense attention: head_dim must be a multiple of 8 and <= 128");
  DenseAttnParams p;
  p.q = (const bf16*)q;
  p.k = (const bf16*)k;
  p.v = (const bf16*)v;
  p.out = (bf16*)out;
  p.key_mask = key_mask;
  p.q_sb = q_strides[0]; p.q_ss = q_strides[1]; p.q_sh = q_strides[2];
  p.k_sb = k_strides[0]; p.k_ss = k_strides[1]; p.k_sh = k_strides[2];
  p.v_sb = v_strides[0]; p.v_ss = v_strides[1]; p.v_sh = v_strides[2];
  p.Sq = Sq; p.Sk = Sk; p.H = H; p.D = D;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int DP = D <= 64 ? 64 : (D <= 80 ? 80 : (D <= 96 ? 96 : 128));
  dim3 grid((Sq + DA_BM - 1) / DA_BM, H, B);
  const int pitch = DP * 2 + 16;
  const int smem = (DA_BM + 4 * DA_BN) * pitch;
  auto launch = [&](auto kern) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    kern<<<grid, DA_THREADS, smem, stream>>>(p);
  };
  if (DP == 64) launch(dense_attn_kernel<64>);
  else if (DP == 80) launch(dense_attn_kernel<80>);
  else if (DP == 96) launch(dense_attn_kernel<96>);
  else launch(dense_attn_kernel<128>);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("dense attention launch: ") + cudaGetErrorString(e));
}

}  // namespace fc
