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

// x [groups, g] bf16 (rows of D values cut into D / g groups).  FAKE: y = decode(encode(x)) in bf16, no codes.
// Otherwise: codes as bytes (INT8, FP8: one per value; INT4 / NF4: one per two values), `scale` [groups] (the
// scale, or the absmax for the 4-bit modes) and, for the asymmetric mode, `zero` [groups].
template <int MODE, bool FAKE>
__global__ void __launch_bounds__(256)
quantize_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale,
                float* __restrict__ zero, bf16* __restrict__ y, long long groups, int g) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int chunks = g >> 3;
  constexpr bool FOUR_BIT = (MODE == QUANT_INT4 || MODE == QUANT_NF4);
  for (long long grp = warp; grp < groups; grp += nwarps) {
    const bf16* src = x + grp * g;
    float v[QMAX_CHUNKS][8];
    float amax = 0.f, lo = INFINITY, hi = -INFINITY;
#pragma unroll
    for (int c = 0; c < QMAX_CHUNKS; ++c) {
      const int idx = lane + 32 * c;
      if (idx < chunks) {
        load8(src + idx * 8, v[c]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          amax = fmaxf(amax, fabsf(v[c][i]));
          lo = fminf(lo, v[c][i]);
          hi = fmaxf(hi, v[c][i]);
        }
      }
    }
    amax = warp_max(amax);
    if (MODE == QUANT_INT8_ASYM) {
      lo = warp_min(lo);
      hi = warp_max(hi);
    }
    float a, z;
    group_params<MODE>(amax, lo, hi, a, z);
    if (!FAKE && lane == 0) {
      scale[grp] = a;
      if (MODE == QUANT_INT8_ASYM) zero[grp] = z;
    }
#pragma unroll
    for (int c = 0; c < QMAX_CHUNKS; ++c) {
      const int idx = lane + 32 * c;
      if (idx < chunks) {
        int code[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) code[i] = encode<MODE>(v[c][i], a, z);
        if (FAKE) {
          float out[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) out[i] = decode<MODE>(code[i], a, z);
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

template <int MODE>
__global__ void __launch_bounds__(256)
dequantize_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scale, const float* __restrict__ zero,
                  bf16* __restrict__ y, long long groups, int g) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int chunks = g >> 3;
  constexpr bool FOUR_BIT = (MODE == QUANT_INT4 || MODE == QUANT_NF4);
  for (long long grp = warp; grp < groups; grp += nwarps) {
    const float a = scale[grp];
    const float z = (MODE == QUANT_INT8_ASYM) ? zero[grp] : 0.f;
    for (int idx = lane; idx < chunks; idx += 32) {
      int code[8];
      if (FOUR_BIT) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(q + grp * (g >> 1) + idx * 4);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t b = (w >> (8 * i)) & 0xFF;
          code[2 * i] = int(b & 0xF);
          code[2 * i + 1] = int(b >> 4);
        }
      } else {
        const uint2 w = *reinterpret_cast<const uint2*>(q + grp * g + idx * 8);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t b0 = (w.x >> (8 * i)) & 0xFF, b1 = (w.y >> (8 * i)) & 0xFF;
          code[i] = (MODE == QUANT_INT8) ? int(int8_t(b0)) : int(b0);
          code[4 + i] = (MODE == QUANT_INT8) ? int(int8_t(b1)) : int(b1);
        }
      }
      float out[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = decode<MODE>(code[i], a, z);
      store8(y + grp * g + idx * 8, out);
    }
  }
}

static int quant_grid(long long groups) {
  const long long blocks = (groups + 7) / 8;                 // 8 warps per block, one group per warp and pass
  return int(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

void launch_quantize(const void* x, void* q, float* scale, float* zero, void* y_fake, long long groups, int g,
                     int mode, cudaStream_t s) {
  if (groups == 0) return;
  if (g % 8 != 0 || g > 32 * QMAX_CHUNKS * 8) throw std::runtime_error("quantize: group size must be a multiple of 8, at most 1024");
  const bf16* xi = (const bf16*)x;
  uint8_t* qo = (uint8_t*)q;
  bf16* yo = (bf16*)y_fake;
  const int grid = quant_grid(groups);
#define FC_QLAUNCH(M)                                                                                       \
  case M:                                                                                                   \
    if (yo != nullptr) quantize_kernel<M, true><<<grid, 256, 0, s>>>(xi, qo, scale, zero, yo, groups, g);     \
    else quantize_kernel<M, false><<<grid, 256, 0, s>>>(xi, qo, scale, zero, yo, groups, g);                 \
    break;
  switch (mode) {
    FC_QLAUNCH(QUANT_INT8)
    FC_QLAUNCH(QUANT_INT8_ASYM)
    FC_QLAUNCH(QUANT_INT4)
    FC_QLAUNCH(QUANT_NF4)
    FC_QLAUNCH(QUANT_FP8_E4M3)
    FC_QLAUNCH(QUANT_FP8_E5M2)
    default: throw std::runtime_error("quantize: unknown mode");
  }
#undef FC_QLAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("quantize launch: ") + cudaGetErrorString(e));
}

void launch_dequantize(const void* q, const float* scale, const float* zero, void* y, long long groups, int g,
                       int mode, cudaStream_t s) {
  if (groups == 0) return;
  if (g % 8 != 0) throw std::runtime_error("dequantize: group size must be a multiple of 8");
  const uint8_t* qi = (const uint8_t*)q;
  bf16* yo = (bf16*)y;
  const int grid = quant_grid(groups);
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
