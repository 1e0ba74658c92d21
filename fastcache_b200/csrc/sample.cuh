// Device code shared by the two sampler kernels (elementwise.cu: one GPU; comm.cu: vocabulary shards on
// several GPUs).  A draw is argmax_j (logit_j / T + Gumbel_j) with the noise a pure function of (seed, row,
// GLOBAL vocabulary index), so a shard can find its own best candidate and the winner over all shards is the
// token that one GPU holding the whole row would have drawn.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace fc {

__device__ __forceinline__ uint32_t sample_mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352dU;
  x ^= x >> 15;
  x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}

__device__ __forceinline__ bool sample_better(float v, int i, float best, int best_i) {
  return v > best || (v == best && i < best_i);
}

// Best (value, global index) of row `row` [V logits, global indices vocab_offset + j, indices >= v_limit are
// padding and never win] for the calling CTA; valid in thread 0 after the call.  `s_val` / `s_idx`: 32 words each.
//
// The value that is compared is logit * (log2 e / T) - log2(-log2 u): the draw logit / T - ln(-ln u) times log2 e
// plus a constant, hence the same winner for one multiply-add and two lg2 per entry.  u = (k + 0.5) / 2^23 with k
// the top 23 bits of the hash: k + 0.5 is exact in fp32, so u stays inside (0, 1) and the noise inside (-2.9, 16.7)
// (with 24 bits the largest k + 0.5 would round up to u = 1 and give that entry infinite noise).
__device__ __forceinline__ void sample_row_best(const __nv_bfloat16* row, int V, int vocab_offset, int v_limit,
                                                float T, uint32_t row_seed, float* s_val, int* s_idx,
                                                float& best, int& best_i) {
  best = -INFINITY;
  best_i = 0x7fffffff;
  const int n = min(V, v_limit - vocab_offset);   // entries that may win (<= 0: none)
  const float scale = T > 0.f ? 1.44269504f / T : 1.0f;
  const uint32_t seed0 = row_seed + uint32_t(vocab_offset);
  int local_i = -1;
  // a thread visits its entries in increasing order, so "strictly greater" keeps the lowest index among equals
  auto consider = [&](float v, int j) {
    if (T > 0.f) {
      const uint32_t r = sample_mix32(seed0 + uint32_t(j));
      const float u = (float(r >> 9) + 0.5f) * (1.0f / 8388608.0f);
      v = fmaf(v, scale, -__log2f(-__log2f(u)));
    }
    if (v > best) {
      best = v;
      local_i = j;
    }
  };
  const bool vec = ((reinterpret_cast<uintptr_t>(row) & 15) == 0);
  const int v8 = (vec && n > 0) ? (n >> 3) : 0;
  for (int c = threadIdx.x; c < v8; c += blockDim.x) {           // 16-byte loads: 8 logits at a time
    const uint4 u = __ldcg(reinterpret_cast<const uint4*>(row) + c);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h2[i]);
      consider(f.x, c * 8 + 2 * i);
      consider(f.y, c * 8 + 2 * i + 1);
    }
  }
  for (int j = v8 * 8 + threadIdx.x; j < n; j += blockDim.x) consider(__bfloat162float(row[j]), j);
  if (local_i >= 0) best_i = vocab_offset + local_i;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (sample_better(ov, oi, best, best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    s_val[warp] = best;
    s_idx[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    best = (lane < int(blockDim.x >> 5)) ? s_val[lane] : -INFINITY;
    best_i = (lane < int(blockDim.x >> 5)) ? s_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (sample_better(ov, oi, best, best_i)) {
        best = ov;
        best_i = oi;
      }
    }
  }
}

__device__ __forceinline__ uint32_t sample_row_seed(uint32_t seed, int b) {
  return sample_mix32(seed ^ (uint32_t(b) * 0x9E3779B9u));
}

}  // namespace fc
