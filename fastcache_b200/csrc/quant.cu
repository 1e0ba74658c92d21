// KV quantisers: per-group absmax quantisation of bf16 rows to INT8 (symmetric / asymmetric), INT4 and NF4
// (two codes per byte, even index in the low nibble) and scaled FP8 (e4m3 / e5m2), their inverses, and the
// quantise-and-restore round trip in one pass ("fake quantisation").
//
// One warp owns one group of `g` consecutive values of a row (g = the whole row for the INT8 and FP8 modes): a
// lane holds up to QMAX_CHUNKS 16-byte pieces in registers, the group statistics (absmax, or min and max) are a
// warp reduction, and the codes go out as packed words.  The op is a single pass over the data: bound by
// bandwidth (2 bytes read, 1 / 0.5 bytes written per value), nothing to put on the tensor cores.
//
// The arithmetic matches the PyTorch statements of fastcache_b200/compress/quant.py operation for operation
// (fp32 division by the scale, round-half-to-even, the same clamps), so codes and scales are bit-identical.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

#include "kernels.h"
#include "ptx.cuh"

namespace fc {

using bf16 = __nv_bfloat16;

constexpr int QMAX_CHUNKS = 4;            // 16-byte pieces per lane: groups of up to 32 * 4 * 8 = 1024 values

__constant__ float c_nf4[16] = {-1.0f, -0.6961928f, -0.52507305f, -0.39491749f, -0.28444138f, -0.18477343f,
                                -0.09105004f, 0.0f, 0.0795803f, 0.1609302f, 0.2461123f, 0.33791524f, 0.44070983f,
                                0.562617f, 0.72295684f, 1.0f};

__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ int nf4_code(float t) {
  int best = 0;
  float bd = fabsf(t - c_nf4[0]);
#pragma unroll
  for (int i = 1; i < 16; ++i) {
    const float d = fabsf(t - c_nf4[i]);
    if (d < bd) {            // the first of equal distances wins, like argmin
      bd = d;
      best = i;
    }
  }
  return best;
}

__device__ __forceinline__ void load8(const bf16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(bf16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]);
  u.y = pack_bf16(f[2], f[3]);
  u.z = pack_bf16(f[4], f[5]);
  u.w = pack_bf16(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// code of one value and the value it stands for; `a` = scale (INT8, FP8) or absmax (INT4, NF4), `z` = zero point
template <int MODE>
__device__ __forceinline__ int encode(float x, float a, float z) {
  if (MODE == QUANT_INT8) return int(fminf(fmaxf(rintf(__fdiv_rn(x, a)), -127.f), 127.f));
  if (MODE == QUANT_INT8_ASYM) return int(fminf(fmaxf(rintf(__fdiv_rn(x - z, a)), 0.f), 255.f));
  if (MODE == QUANT_INT4) return int(fminf(fmaxf(rintf(__fdiv_rn(x, a) * 7.0f), -8.f), 7.f)) + 8;
  if (MODE == QUANT_NF4) return nf4_code(__fdiv_rn(x, a));
  if (MODE == QUANT_FP8_E4M3) return int(__nv_cvt_float_to_fp8(__fdiv_rn(x, a), __NV_SATFINITE, __NV_E4M3));
  return int(__nv_cvt_float_to_fp8(__fdiv_rn(x, a), __NV_SATFINITE, __NV_E5M2));
}
template <int MODE>
__device__ __forceinline__ float decode(int q, float a, float z) {
  if (MODE == QUANT_INT8) return float(q) * a;
  if (MODE == QUANT_INT8_ASYM) return __fadd_rn(__fmul_rn(float(q), a), z);   // two roundings, like the tensor ops
  if (MODE == QUANT_INT4) return __fdiv_rn(float(q) - 8.0f, 7.0f) * a;
  if (MODE == QUANT_NF4) return c_nf4[q] * a;
  const __nv_fp8_interpretation_t kind = (MODE == QUANT_FP8_E4M3) ? __NV_E4M3 : __NV_E5M2;
  const __half_raw h = __nv_cvt_fp8_to_halfraw(__nv_fp8_storage_t(q), kind);
  return __half2float(__half(h)) * a;
}

// group statistics of the values a warp holds -> (a, z) as `encode` wants them
template <int MODE>
__device__ __forceinline__ void group_params(float amax, float lo, float hi, float& a, float& z) {
  z = 0.f;
  if (MODE == QUANT_INT8) a = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
  else if (MODE == QUANT_INT8_ASYM) {
    a = fmaxf(__fdiv_rn(hi - lo, 255.0f), 1e-8f);
    z = lo;
  } else if (MODE == QUANT_INT4 || MODE == QUANT_NF4) a = fmaxf(amax, 1e-8f);
  else a = __fdiv_rn(fmaxf(amax, 1e-8f), MODE == QUANT_FP8_E4M3 ? 448.0f : 57344.0f);
}

// Lanes per group: a group of g values is g / 8 pieces of 16 bytes; W = the next power of two (at most 32) lanes
// share one group, 32 / W groups sit side by side in a warp and QU such batches are in flight per iteration, so
// every lane has QU independent 16-byte loads outstanding (a 128-value group uses 16 lanes: without this half of
// every warp would idle and each lane would wait for one load at a time).  Groups longer than 256 values give a
// lane several pieces (W = 32, up to QMAX_CHUNKS).
constexpr int QU = 4;

template <int W>
__device__ __forceinline__ float sub_max(float v) {
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int W>
__device__ __forceinline__ float sub_min(float v) {
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// the 16 restored values of the two 4-bit modes, in shared memory (an index that differs between lanes reads a
// __constant__ table one lane at a time)
template <int MODE>
__device__ __forceinline__ void fill_table4(float* s_tab) {
  if (threadIdx.x < 16)
    s_tab[threadIdx.x] = (MODE == QUANT_NF4) ? c_nf4[threadIdx.x] : __fdiv_rn(float(int(threadIdx.x)) - 8.0f, 7.0f);
  __syncthreads();
}
// NF4 code by bisection over the 15 midpoints between neighbouring table entries: the entry nearest to t, the
// lower one at a midpoint (what argmin over the distances gives)
__device__ __forceinline__ int nf4_code_fast(float t, const float* s_mid) {
  int c = (t > s_mid[7]) ? 8 : 0;
  c += (t > s_mid[c + 3]) ? 4 : 0;
  c += (t > s_mid[c + 1]) ? 2 : 0;
  c += (t > s_mid[c]) ? 1 : 0;
  return c;
}

// x [groups, g] bf16 (rows of D values cut into D / g groups).  FAKE: y = decode(encode(x)) in bf16, no codes.
// Otherwise: codes as bytes (INT8, FP8: one per value; INT4 / NF4: one per two values), `scale` [groups] (the
// scale, or the absmax for the 4-bit modes) and, for the asymmetric mode, `zero` [groups].
template <int MODE, bool FAKE, int W>
__global__ void __launch_bounds__(256)
quantize_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale,
                float* __restrict__ zero, bf16* __restrict__ y, long long groups, int g) {
  __shared__ float s_tab[16];
  __shared__ float s_mid[16];
  constexpr bool FOUR_BIT = (MODE == QUANT_INT4 || MODE == QUANT_NF4);
  if (FOUR_BIT) {
    if (MODE == QUANT_NF4 && threadIdx.x < 15) s_mid[threadIdx.x] = 0.5f * (c_nf4[threadIdx.x] + c_nf4[threadIdx.x + 1]);
    fill_table4<MODE>(s_tab);
  }
  const int lane = threadIdx.x & 31;
  const int sub = lane / W, l = lane % W;
  constexpr int GPW = 32 / W;                                    // groups per warp and batch
  constexpr int CH = (W == 32) ? QMAX_CHUNKS : 1;                // 16-byte pieces per lane and group
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int chunks = g >> 3;
  for (long long g0 = warp * (GPW * QU); g0 < groups; g0 += nwarps * (GPW * QU)) {
    float v[QU][CH][8];
    float amax[QU], lo[QU], hi[QU];
#pragma unroll
    for (int u = 0; u < QU; ++u) {
      const long long grp = g0 + u * GPW + sub;
      amax[u] = 0.f;
      lo[u] = INFINITY;
      hi[u] = -INFINITY;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int idx = l + W * c;
        if (grp < groups && idx < chunks) load8(x + grp * g + idx * 8, v[u][c]);
      }
    }
#pragma unroll
    for (int u = 0; u < QU; ++u) {
      const long long grp = g0 + u * GPW + sub;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int idx = l + W * c;
        if (grp < groups && idx < chunks) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            amax[u] = fmaxf(amax[u], fabsf(v[u][c][i]));
            lo[u] = fminf(lo[u], v[u][c][i]);
            hi[u] = fmaxf(hi[u], v[u][c][i]);
          }
        }
      }
      amax[u] = sub_max<W>(amax[u]);
      if (MODE == QUANT_INT8_ASYM) {
        lo[u] = sub_min<W>(lo[u]);
        hi[u] = sub_max<W>(hi[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < QU; ++u) {
      const long long grp = g0 + u * GPW + sub;
      if (grp >= groups) continue;
      float a, z;
      group_params<MODE>(amax[u], lo[u], hi[u], a, z);
      if (!FAKE && l == 0) {
        scale[grp] = a;
        if (MODE == QUANT_INT8_ASYM) zero[grp] = z;
      }
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int idx = l + W * c;
        if (idx >= chunks) continue;
        int code[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          code[i] = (MODE == QUANT_NF4) ? nf4_code_fast(__fdiv_rn(v[u][c][i], a), s_mid) : encode<MODE>(v[u][c][i], a, z);
        if (FAKE) {
          float out[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) out[i] = FOUR_BIT ? s_tab[code[i]] * a : decode<MODE>(code[i], a, z);
          store8(y + grp * g + idx * 8, out);
        } else if (FOUR_BIT) {
          uint32_t w = 0;
#pragma unroll
          for (int i = 0; i < 4; ++i) w |= uint32_t((code[2 * i] & 0xF) | ((code[2 * i + 1] & 0xF) << 4)) << (8 * i);
          *reinterpret_cast<uint32_t*>(q + grp * (g >> 1) + idx * 4) = w;
        } else {
          uint2 w = make_uint2(0, 0);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            w.x |= uint32_t(code[i] & 0xFF) << (8 * i);
            w.y |= uint32_t(code[4 + i] & 0xFF) << (8 * i);
          }
          *reinterpret_cast<uint2*>(q + grp * g + idx * 8) = w;
        }
      }
    }
  }
}

// one thread per 16-byte piece of the output, grid-stride: nothing is shared between the pieces of a group but its
// scale, so no warp-level structure is needed
template <int MODE>
__global__ void __launch_bounds__(256)
dequantize_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scale, const float* __restrict__ zero,
                  bf16* __restrict__ y, long long groups, int g) {
  __shared__ float s_tab[16];
  constexpr bool FOUR_BIT = (MODE == QUANT_INT4 || MODE == QUANT_NF4);
  if (FOUR_BIT) fill_table4<MODE>(s_tab);
  const int chunks = g >> 3;
  const long long total = groups * chunks;
  for (long long p = blockIdx.x * (long long)blockDim.x + threadIdx.x; p < total;
       p += (long long)gridDim.x * blockDim.x) {
    const long long grp = p / chunks;
    const int idx = int(p - grp * chunks);
    const float a = scale[grp];
    const float z = (MODE == QUANT_INT8_ASYM) ? zero[grp] : 0.f;
    float out[8];
    if (FOUR_BIT) {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(q + grp * (g >> 1) + idx * 4);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t b = (w >> (8 * i)) & 0xFF;
        out[2 * i] = s_tab[b & 0xF] * a;
        out[2 * i + 1] = s_tab[b >> 4] * a;
      }
    } else {
      const uint2 w = *reinterpret_cast<const uint2*>(q + grp * g + idx * 8);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t b0 = (w.x >> (8 * i)) & 0xFF, b1 = (w.y >> (8 * i)) & 0xFF;
        out[i] = decode<MODE>((MODE == QUANT_INT8) ? int(int8_t(b0)) : int(b0), a, z);
        out[4 + i] = decode<MODE>((MODE == QUANT_INT8) ? int(int8_t(b1)) : int(b1), a, z);
      }
    }
    store8(y + grp * g + idx * 8, out);
  }
}

static int quant_grid(long long work_items, int per_block) {
  const long long blocks = (work_items + per_block - 1) / per_block;
  return int(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

template <int MODE, int W>
static void launch_quantize_w(const bf16* x, uint8_t* q, float* scale, float* zero, bf16* y, long long groups, int g,
                              cudaStream_t s) {
  const int grid = quant_grid(groups, 8 * (32 / W) * QU);          // groups per block and iteration
  if (y != nullptr) quantize_kernel<MODE, true, W><<<grid, 256, 0, s>>>(x, q, scale, zero, y, groups, g);
  else quantize_kernel<MODE, false, W><<<grid, 256, 0, s>>>(x, q, scale, zero, y, groups, g);
}
template <int MODE>
static void launch_quantize_m(const bf16* x, uint8_t* q, float* scale, float* zero, bf16* y, long long groups, int g,
                              cudaStream_t s) {
  const int chunks = g >> 3;
  if (chunks <= 4) launch_quantize_w<MODE, 4>(x, q, scale, zero, y, groups, g, s);
  else if (chunks <= 8) launch_quantize_w<MODE, 8>(x, q, scale, zero, y, groups, g, s);
  else if (chunks <= 16) launch_quantize_w<MODE, 16>(x, q, scale, zero, y, groups, g, s);
  else launch_quantize_w<MODE, 32>(x, q, scale, zero, y, groups, g, s);
}

void launch_quantize(const void* x, void* q, float* scale, float* zero, void* y_fake, long long groups, int g,
                     int mode, cudaStream_t s) {
  if (groups == 0) return;
  if (g % 8 != 0 || g > 32 * QMAX_CHUNKS * 8) throw std::runtime_error("quantize: group size must be a multiple of 8, at most 1024");
  const bf16* xi = (const bf16*)x;
  uint8_t* qo = (uint8_t*)q;
  bf16* yo = (bf16*)y_fake;
  switch (mode) {
    case QUANT_INT8: launch_quantize_m<QUANT_INT8>(xi, qo, scale, zero, yo, groups, g, s); break;
    case QUANT_INT8_ASYM: launch_quantize_m<QUANT_INT8_ASYM>(xi, qo, scale, zero, yo, groups, g, s); break;
    case QUANT_INT4: launch_quantize_m<QUANT_INT4>(xi, qo, scale, zero, yo, groups, g, s); break;
    case QUANT_NF4: launch_quantize_m<QUANT_NF4>(xi, qo, scale, zero, yo, groups, g, s); break;
    case QUANT_FP8_E4M3: launch_quantize_m<QUANT_FP8_E4M3>(xi, qo, scale, zero, yo, groups, g, s); break;
    case QUANT_FP8_E5M2: launch_quantize_m<QUANT_FP8_E5M2>(xi, qo, scale, zero, yo, groups, g, s); break;
    default: throw std::runtime_error("quantize: unknown mode");
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("quantize launch: ") + cudaGetErrorString(e));
}

void launch_dequantize(const void* q, const float* scale, const float* zero, void* y, long long groups, int g,
                       int mode, cudaStream_t s) {
  if (groups == 0) return;
  if (g % 8 != 0) throw std::runtime_error("dequantize: group size must be a multiple of 8");
  const uint8_t* qi = (const uint8_t*)q;
  bf16* yo = (bf16*)y;
  const int grid = quant_grid(groups * (g >> 3), 256);
  switch (mode) {
    case QUANT_INT8: dequantize_kernel<QUANT_INT8><<<grid, 256, 0, s>>>(qi, scale, zero, yo, groups, g); break;
    case QUANT_INT8_ASYM: dequantize_kernel<QUANT_INT8_ASYM><<<grid, 256, 0, s>>>(qi, scale, zero, yo, groups, g); break;
    case QUANT_INT4: dequantize_kernel<QUANT_INT4><<<grid, 256, 0, s>>>(qi, scale, zero, yo, groups, g); break;
    case QUANT_NF4: dequantize_kernel<QUANT_NF4><<<grid, 256, 0, s>>>(qi, scale, zero, yo, groups, g); break;
    case QUANT_FP8_E4M3: dequantize_kernel<QUANT_FP8_E4M3><<<grid, 256, 0, s>>>(qi, scale, zero, yo, groups, g); break;
    case QUANT_FP8_E5M2: dequantize_kernel<QUANT_FP8_E5M2><<<grid, 256, 0, s>>>(qi, scale, zero, yo, groups, g); break;
    default: throw std::runtime_error("dequantize: unknown mode");
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("dequantize launch: ") + cudaGetErrorString(e));
}

}  // namespace fc
