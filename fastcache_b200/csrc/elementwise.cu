// Bandwidth-bound ops: RMSNorm / add+RMSNorm / LayerNorm, SwiGLU gate, embedding
// gather, fused q/k-norm + rotary + paged KV store, and the sampler.  All bf16
// in/out with fp32 math; rows are held in registers between the statistics pass
// and the scaling pass so each element is read once.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <algorithm>
#include <stdexcept>
#include <string>

#include "kernels.h"
#include "launch.h"
#include "ptx.cuh"
#include "sample.cuh"

namespace fc {

using bf16 = __nv_bfloat16;

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_CHUNKS = 4;   // 16-byte chunks per thread: rows up to 256 * 4 * 8 = 8192 elements

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]);
  u.y = pack_bf16(f[2], f[3]);
  u.z = pack_bf16(f[4], f[5]);
  u.w = pack_bf16(f[6], f[7]);
  return u;
}

// y = rms_norm(x [+ residual]) * w ; if residual != nullptr it is updated in place with x + residual.
// One block per row; H % 8 == 0, H <= 8192; x is bf16 (fp32 split-K partial sums go through partials.cu).
template <bool ADD>
__global__ void __launch_bounds__(NORM_THREADS)
rms_norm_kernel(const bf16* __restrict__ x, bf16* __restrict__ residual, const bf16* __restrict__ w,
                bf16* __restrict__ y, int H, float eps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const long long row = blockIdx.x;
  const int chunks = H >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  uint4* rr = ADD ? reinterpret_cast<uint4*>(residual + row * H) : nullptr;
  float v[NORM_MAX_CHUNKS][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
    const int idx = threadIdx.x + c * NORM_THREADS;
    if (idx < chunks) {
      unpack8(xr[idx], v[c]);
      if (ADD) {
        float r[8];
        unpack8(rr[idx], r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] += r[i];
        const uint4 s = pack8(v[c]);
        rr[idx] = s;
        unpack8(s, v[c]);            // normalise the bf16-rounded sum, like the PyTorch statement
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[c][i] * v[c][i];
    }
  }
  const float tot = block_sum(ss, red);
  const float inv = rsqrtf(tot / float(H) + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * H);
#pragma unroll
  for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
    const int idx = threadIdx.x + c * NORM_THREADS;
    if (idx < chunks) {
      float g[8], o[8];
      unpack8(wr[idx], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = __bfloat162float(__float2bfloat16(v[c][i] * inv)) * g[i];
      yr[idx] = pack8(o);
    }
  }
}

__global__ void __launch_bounds__(NORM_THREADS)
layer_norm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ b,
                  bf16* __restrict__ y, int H, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int chunks = H >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  float v[NORM_MAX_CHUNKS][8];
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
    const int idx = threadIdx.x + c * NORM_THREADS;
    if (idx < chunks) {
      unpack8(xr[idx], v[c]);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += v[c][i];
    }
  }
  const float mean = block_sum(s, red) / float(H);
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
    const int idx = threadIdx.x + c * NORM_THREADS;
    if (idx < chunks) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = v[c][i] - mean;
        ss += d * d;
      }
    }
  }
  const float inv = rsqrtf(block_sum(ss, red) / float(H) + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const uint4* br = reinterpret_cast<const uint4*>(b);
  uint4* yr = reinterpret_cast<uint4*>(y + row * H);
#pragma unroll
  for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
    const int idx = threadIdx.x + c * NORM_THREADS;
    if (idx < chunks) {
      float g[8], bb[8], o[8];
      unpack8(wr[idx], g);
      unpack8(br[idx], bb);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = (v[c][i] - mean) * inv * g[i] + bb[i];
      yr[idx] = pack8(o);
    }
  }
}

// y[t, i] = silu(x[t, i]) * x[t, I + i]
__global__ void silu_and_mul_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long T, int I) {
  const int chunks = I >> 3;
  const long long total = T * chunks;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / chunks;
    const int c = int(idx - t * chunks);
    const uint4* row = reinterpret_cast<const uint4*>(x + t * 2 * I);
    float g[8], u[8], o[8];
    unpack8(row[c], g);
    unpack8(row[chunks + c], u);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
    reinterpret_cast<uint4*>(y + t * I)[c] = pack8(o);
  }
}

// out[t, :] = (vocab_start <= ids[t] < vocab_start + V) ? weight[ids[t] - vocab_start, :] : 0
__global__ void embedding_kernel(const long long* __restrict__ ids, const bf16* __restrict__ weight,
                                 bf16* __restrict__ out, int T, int H, int V, int vocab_start) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const long long id = ids[t] - vocab_start;
  const int chunks = H >> 3;
  uint4* o = reinterpret_cast<uint4*>(out + (long long)t * H);
  if (id < 0 || id >= V) {
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) o[c] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(weight + id * H);
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) o[c] = src[c];
}

// One warp per (token, head).  Heads [0, Hq) are queries (normed, rotated, written to q_out),
// [Hq, Hq+Hkv) keys (normed, rotated, stored in the pool), the rest values (stored).
__global__ void __launch_bounds__(128)
rope_qknorm_store_kernel(const bf16* __restrict__ qkv, const long long* __restrict__ positions,
                         const float* __restrict__ cos_sin, const bf16* __restrict__ q_w,
                         const bf16* __restrict__ k_w, bf16* __restrict__ q_out, bf16* __restrict__ k_cache,
                         bf16* __restrict__ v_cache, const int* __restrict__ slots, int T, int Hq, int Hkv,
                         int D, float eps, long long num_slots, int block_size, uint32_t* status) {
  const int heads = Hq + 2 * Hkv;
  const long long wid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)T * heads) return;
  const int t = int(wid / heads);
  const int h = int(wid - (long long)t * heads);
  const bf16* src = qkv + (long long)t * heads * D + (long long)h * D;
  const int half = D >> 1;
  long long slot = -1;
  if (h >= Hq && slots != nullptr) {
    slot = slots[t];
    if (slot >= num_slots) {
      report(status, ST_BAD_INDEX);
      slot = -1;
    }
  }
  if (h >= Hq + Hkv) {            // value head: plain copy into the pool
    if (slot < 0) return;
    bf16* dst = v_cache + (((slot / block_size) * Hkv + (h - Hq - Hkv)) * block_size + slot % block_size) * D;
    for (int i = lane; i < (D >> 3); i += 32)
      reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    return;
  }
  const bool is_q = h < Hq;
  const bf16* nw = is_q ? q_w : k_w;
  if (!is_q && slot < 0 && slots != nullptr) return;
  if (D == 128) {
    // fast path: each lane owns the pairs (2l, 2l+1) of the low half and their partners in the high half
    const __nv_bfloat162* s2 = reinterpret_cast<const __nv_bfloat162*>(src);
    float2 a = __bfloat1622float2(s2[lane]), b = __bfloat1622float2(s2[32 + lane]);
    if (nw != nullptr) {
      const float inv = rsqrtf(warp_sum(a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y) / 128.f + eps);
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(nw);
      const float2 wa = __bfloat1622float2(w2[lane]), wb = __bfloat1622float2(w2[32 + lane]);
      auto rn = [](float v) { return __bfloat162float(__float2bfloat16(v)); };
      a.x = rn(rn(a.x * inv) * wa.x);
      a.y = rn(rn(a.y * inv) * wa.y);
      b.x = rn(rn(b.x * inv) * wb.x);
      b.y = rn(rn(b.y * inv) * wb.y);
    }
    const float2* cs2 = reinterpret_cast<const float2*>(cos_sin + positions[t] * 128);
    const float2 c = cs2[lane], s = cs2[32 + lane];
    __nv_bfloat162* d2 = reinterpret_cast<__nv_bfloat162*>(
        is_q ? (q_out + ((long long)t * Hq + h) * 128)
             : (k_cache + (((slot / block_size) * Hkv + (h - Hq)) * block_size + slot % block_size) * 128));
    d2[lane] = __floats2bfloat162_rn(a.x * c.x - b.x * s.x, a.y * c.y - b.y * s.y);
    d2[32 + lane] = __floats2bfloat162_rn(b.x * c.x + a.x * s.x, b.y * c.y + a.y * s.y);
    return;
  }
  // pairs (p, p + half), p = lane, lane + 32, ...   (D <= 256)
  float lo[4], hi[4];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int p = lane + 32 * j;
    if (p < half) {
      lo[j] = __bfloat162float(src[p]);
      hi[j] = __bfloat162float(src[p + half]);
      ss += lo[j] * lo[j] + hi[j] * hi[j];
    }
  }
  if (nw != nullptr) {
    const float inv = rsqrtf(warp_sum(ss) / float(D) + eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = lane + 32 * j;
      if (p < half) {
        lo[j] = __bfloat162float(__float2bfloat16(lo[j] * inv)) * __bfloat162float(nw[p]);
        hi[j] = __bfloat162float(__float2bfloat16(hi[j] * inv)) * __bfloat162float(nw[p + half]);
        // the PyTorch statement rounds the normed head to bf16 before the rotation
        lo[j] = __bfloat162float(__float2bfloat16(lo[j]));
        hi[j] = __bfloat162float(__float2bfloat16(hi[j]));
      }
    }
  }
  const float* cs = cos_sin + positions[t] * D;
  bf16* dst = is_q ? (q_out + ((long long)t * Hq + h) * D) : (k_cache + (((slot / block_size) * Hkv + (h - Hq)) * block_size + slot % block_size) * D);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int p = lane + 32 * j;
    if (p < half) {
      const float c = cs[p], s = cs[p + half];
      dst[p] = __float2bfloat16(lo[j] * c - hi[j] * s);
      dst[p + half] = __float2bfloat16(hi[j] * c + lo[j] * s);
    }
  }
}

// head_dim 128: eight lanes per (token, head), each lane owns 8 consecutive elements of the low
// half and their rotation partners in the high half (two 16-byte loads, two 16-byte stores).
__global__ void __launch_bounds__(256)
rope_qknorm_store_d128_kernel(const bf16* __restrict__ qkv, const long long* __restrict__ positions,
                              const float* __restrict__ cos_sin, const bf16* __restrict__ q_w,
                              const bf16* __restrict__ k_w, bf16* __restrict__ q_out, bf16* __restrict__ k_cache,
                              bf16* __restrict__ v_cache, const int* __restrict__ slots, int T, int Hq, int Hkv,
                              float eps, long long num_slots, int block_size, uint32_t* status,
                              const float* __restrict__ partial, int splits, long long split_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int heads = Hq + 2 * Hkv;
  const long long gid = (blockIdx.x * 256ll + threadIdx.x) >> 3;
  const int j = threadIdx.x & 7;
  const bool active = gid < (long long)T * heads;
  const long long g = active ? gid : 0;
  const int t = int(g / heads);
  const int h = int(g - (long long)t * heads);
  uint4 ulo, uhi;
  if (partial != nullptr) {
    // qkv is still the split-K partial sums of its GEMM ([splits, T, heads * 128] fp32): reduce them here and
    // round to bf16 as the GEMM epilogue would have
    const float* p0 = partial + ((long long)t * heads + h) * 128 + 8 * j;
    float a[8], b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = b[i] = 0.f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
      const float4* ps = reinterpret_cast<const float4*>(p0 + s * split_stride);
      const float4 l0 = __ldcg(ps), l1 = __ldcg(ps + 1), h0 = __ldcg(ps + 16), h1 = __ldcg(ps + 17);
      a[0] += l0.x; a[1] += l0.y; a[2] += l0.z; a[3] += l0.w;
      a[4] += l1.x; a[5] += l1.y; a[6] += l1.z; a[7] += l1.w;
      b[0] += h0.x; b[1] += h0.y; b[2] += h0.z; b[3] += h0.w;
      b[4] += h1.x; b[5] += h1.y; b[6] += h1.z; b[7] += h1.w;
    }
    ulo = pack8(a);
    uhi = pack8(b);
  } else {
    const uint4* src = reinterpret_cast<const uint4*>(qkv + ((long long)t * heads + h) * 128);
    ulo = src[j];
    uhi = src[8 + j];
  }
  long long slot = -1;
  if (h >= Hq && slots != nullptr) {
    slot = slots[t];
    if (slot >= num_slots) {
      report(status, ST_BAD_INDEX);
      slot = -1;
    }
  }
  float lo[8], hi[8];
  unpack8(ulo, lo);
  unpack8(uhi, hi);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss += lo[i] * lo[i] + hi[i] * hi[i];
  // every lane of the warp takes part (the 8-lane groups of a warp may sit on different heads)
  ss += __shfl_xor_sync(0xffffffffu, ss, 1);
  ss += __shfl_xor_sync(0xffffffffu, ss, 2);
  ss += __shfl_xor_sync(0xffffffffu, ss, 4);
  if (!active) return;
  if (h >= Hq + Hkv) {            // value head: plain copy into the pool
    if (slot < 0) return;
    uint4* dst = reinterpret_cast<uint4*>(
        v_cache + (((slot / block_size) * Hkv + (h - Hq - Hkv)) * block_size + slot % block_size) * 128);
    dst[j] = ulo;
    dst[8 + j] = uhi;
    return;
  }
  const bool is_q = h < Hq;
  if (!is_q && slot < 0) return;
  const bf16* nw = is_q ? q_w : k_w;
  if (nw != nullptr) {
    const float inv = rsqrtf(ss / 128.f + eps);
    float wl[8], wh[8];
    unpack8(reinterpret_cast<const uint4*>(nw)[j], wl);
    unpack8(reinterpret_cast<const uint4*>(nw)[8 + j], wh);
    auto rn = [](float v) { return __bfloat162float(__float2bfloat16(v)); };
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      lo[i] = rn(rn(lo[i] * inv) * wl[i]);
      hi[i] = rn(rn(hi[i] * inv) * wh[i]);
    }
  }
  const float4* cs = reinterpret_cast<const float4*>(cos_sin + positions[t] * 128);
  const float4 c0 = cs[2 * j], c1 = cs[2 * j + 1], s0 = cs[16 + 2 * j], s1 = cs[16 + 2 * j + 1];
  const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  uint4 olo, ohi;
  uint32_t* pl = reinterpret_cast<uint32_t*>(&olo);
  uint32_t* ph = reinterpret_cast<uint32_t*>(&ohi);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    pl[i] = pack_bf16(lo[2 * i] * c[2 * i] - hi[2 * i] * s[2 * i],
                      lo[2 * i + 1] * c[2 * i + 1] - hi[2 * i + 1] * s[2 * i + 1]);
    ph[i] = pack_bf16(hi[2 * i] * c[2 * i] + lo[2 * i] * s[2 * i],
                      hi[2 * i + 1] * c[2 * i + 1] + lo[2 * i + 1] * s[2 * i + 1]);
  }
  uint4* dst = reinterpret_cast<uint4*>(
      is_q ? (q_out + ((long long)t * Hq + h) * 128)
           : (k_cache + (((slot / block_size) * Hkv + (h - Hq)) * block_size + slot % block_size) * 128));
  dst[j] = olo;
  dst[8 + j] = ohi;
}

// ------------------------------------------------------------------- sampler
// token[b] = argmax_j logits[b, j] / T_b + Gumbel_j   (plain argmax when T_b == 0).
// argmax(softmax(l / T) / E) with E ~ Exp(1) is the same draw: log p_j - log E_j.
// out has B + 1 entries: the last one receives the device status word, so the host learns about a wait that
// ran out (or a bad index) with the tokens it reads back every step anyway.
// One row is shared by a cluster of SAMPLE_SPLIT CTAs (a quarter of the vocabulary each, so that 128 rows fill
// 148 SMs several times over instead of leaving 20 idle and the rest with one CTA); the CTAs hand their
// candidates to the first one through distributed shared memory.  The draw does not depend on the split: the
// noise is a function of the global index and ties go to the lower index.
constexpr int SAMPLE_SPLIT = 4;
constexpr int SAMPLE_THREADS = 512;

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const bf16* __restrict__ logits, const float* __restrict__ temps, long long* __restrict__ out,
              int V, long long ld, uint32_t seed, int vocab_offset, int v_limit, const uint32_t* status) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ __align__(8) uint2 s_cand[SAMPLE_SPLIT];   // (value bits, global index) by CTA of the cluster; used in CTA 0
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;
  const uint32_t part = cluster_ctarank(), parts = cluster_nctarank();
  // slices start at multiples of 8 entries: the 16-byte loads of a slice stay aligned when the row is
  const int per = ((V + int(parts) * 8 - 1) / (int(parts) * 8)) * 8;
  const int j0 = min(V, int(part) * per), j1 = min(V, j0 + per);
  float best;
  int best_i;
  sample_row_best(logits + (long long)b * ld + j0, j1 - j0, vocab_offset + j0, v_limit, temps[b],
                  sample_row_seed(seed, b), s_val, s_idx, best, best_i);
  if (threadIdx.x == 0) {
    const uint32_t cell = cluster_map_shared(smem_u32(&s_cand[part]), 0);
    asm volatile("st.shared::cluster.v2.b32 [%0], {%1, %2};" ::"r"(cell), "r"(__float_as_uint(best)), "r"(best_i)
                 : "memory");
  }
  cluster_sync();
  if (part == 0 && threadIdx.x == 0) {
    best = -INFINITY;
    best_i = 0x7fffffff;
    for (uint32_t r = 0; r < parts; ++r) {
      const float v = __uint_as_float(s_cand[r].x);
      const int i = int(s_cand[r].y);
      if (sample_better(v, i, best, best_i)) {
        best = v;
        best_i = i;
      }
    }
    // a row without a single admissible entry (every index >= v_limit) yields index 0x7fffffff
    out[b] = best_i;
    if (b == 0 && status != nullptr)
      out[gridDim.x] = (long long)(*reinterpret_cast<const volatile uint32_t*>(status) & ST_CODE_MASK);
  }
}

// ================================================================= launchers
void launch_rms_norm(const void* x, void* residual, const void* w, void* y, long long T, int H, float eps,
                     cudaStream_t s) {
  if (T == 0) return;
  if (residual != nullptr)
    launch_pdl(PDL_NORM, rms_norm_kernel<true>, dim3((unsigned)T), dim3(NORM_THREADS), 0, s, (const bf16*)x, (bf16*)residual,
               (const bf16*)w, (bf16*)y, H, eps);
  else
    launch_pdl(PDL_NORM, rms_norm_kernel<false>, dim3((unsigned)T), dim3(NORM_THREADS), 0, s, (const bf16*)x, (bf16*)nullptr,
               (const bf16*)w, (bf16*)y, H, eps);
}

void launch_layer_norm(const void* x, const void* w, const void* b, void* y, long long T, int H, float eps,
                       cudaStream_t s) {
  if (T == 0) return;
  layer_norm_kernel<<<(unsigned)T, NORM_THREADS, 0, s>>>((const bf16*)x, (const bf16*)w, (const bf16*)b, (bf16*)y,
                                                         H, eps);
}

void launch_silu_and_mul(const void* x, void* y, long long T, int I, cudaStream_t s) {
  if (T == 0) return;
  const long long total = T * (I >> 3);
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148 * 16);
  silu_and_mul_kernel<<<blocks, 256, 0, s>>>((const bf16*)x, (bf16*)y, T, I);
}

void launch_embedding(const void* ids, const void* weight, void* out, int T, int H, int V, int vocab_start,
                      cudaStream_t s) {
  if (T == 0) return;
  launch_pdl(PDL_EMBEDDING, embedding_kernel, dim3(T), dim3(128), 0, s, (const long long*)ids, (const bf16*)weight, (bf16*)out, T, H,
             V, vocab_start);
}

void launch_rope_qknorm_store(const void* qkv, const void* positions, const void* cos_sin, const void* q_w,
                              const void* k_w, void* q_out, void* k_cache, void* v_cache, const void* slots, int T,
                              int Hq, int Hkv, int D, float eps, long long num_slots, int block_size,
                              uint32_t* status, cudaStream_t s, const float* partial, int splits,
                              long long split_stride) {
  if (T == 0) return;
  const long long warps = (long long)T * (Hq + 2 * Hkv);
  if (D == 128 && slots != nullptr) {
    launch_pdl(PDL_ROPE, rope_qknorm_store_d128_kernel, dim3((unsigned)((warps + 31) / 32)), dim3(256), 0, s,
               (const bf16*)qkv, (const long long*)positions, (const float*)cos_sin, (const bf16*)q_w,
               (const bf16*)k_w, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, (const int*)slots, T, Hq, Hkv, eps,
               num_slots, block_size, status, partial, splits, split_stride);
    return;
  }
  if (partial != nullptr) throw std::runtime_error("rope from split-K partial sums needs head_dim 128 and a slot map");
  const long long blocks = (warps + 3) / 4;
  rope_qknorm_store_kernel<<<(unsigned)blocks, 128, 0, s>>>(
      (const bf16*)qkv, (const long long*)positions, (const float*)cos_sin, (const bf16*)q_w, (const bf16*)k_w,
      (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, (const int*)slots, T, Hq, Hkv, D, eps, num_slots, block_size,
      status);
}

void launch_sample(const void* logits, const void* temps, void* out, int B, int V, long long ld, uint32_t seed,
                   cudaStream_t s, int vocab_offset, int v_limit, const uint32_t* status) {
  if (B == 0) return;
  const cudaError_t e =
      launch_pdl_cluster(PDL_SAMPLE, sample_kernel, dim3(B, SAMPLE_SPLIT), dim3(SAMPLE_THREADS), 0, s, SAMPLE_SPLIT,
                         (const bf16*)logits, (const float*)temps, (long long*)out, V, ld, seed, vocab_offset,
                         v_limit < 0 ? vocab_offset + V : v_limit, status);
  // a cluster that the stream's SM set cannot place is a launch error, not a kernel that ran: say so here
  if (e != cudaSuccess) throw std::runtime_error(std::string("sampler launch: ") + cudaGetErrorString(e));
}

}  // namespace fc
