// Consumers of split-K partial sums.  The decode-size GEMM (gemm_skinny.cu) leaves fp32
// partials [splits, M, N] in scratch when it splits K; instead of a separate reduction
// pass, the op that reads the GEMM result sums them while it does its own work:
//   * add_rms_norm_partials: y = sum_s partial[s] (+ bias); residual += y; out = RMSNorm(residual)
//   * silu_mul_partials:     g|u = sum_s partial[s]; out = silu(g) * u
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "kernels.h"
#include "launch.h"
#include "ptx.cuh"

namespace fc {

using bf16 = __nv_bfloat16;

constexpr int PN_THREADS = 256;
constexpr int PN_MAX_CHUNKS = 4;        // 8-element chunks per thread: H <= 8192

__global__ void __launch_bounds__(PN_THREADS)
add_rms_norm_partials_kernel(const float* __restrict__ partial, int splits, long long split_stride,
                             const bf16* __restrict__ bias, bf16* __restrict__ residual,
                             const bf16* __restrict__ w, bf16* __restrict__ y, int H, float eps) {
  __shared__ float red[PN_THREADS / 32];
  pdl_launch_dependents();
  pdl_wait();
  const long long row = blockIdx.x;
  const int chunks = H >> 3;
  float v[PN_MAX_CHUNKS][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < PN_MAX_CHUNKS; ++c) {
    const int idx = threadIdx.x + c * PN_THREADS;
    if (idx < chunks) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      const float* p0 = partial + row * H + idx * 8;
#pragma unroll 4
      for (int s = 0; s < splits; ++s) {          // loads of four splits in flight, summed in split order
        const float4 a = __ldcg(reinterpret_cast<const float4*>(p0 + s * split_stride));
        const float4 b = __ldcg(reinterpret_cast<const float4*>(p0 + s * split_stride) + 1);
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
      }
      uint4* rp = reinterpret_cast<uint4*>(residual + row * H + idx * 8);
      const uint4 ru = *rp;
      const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&ru);
      uint4 su;
      uint32_t* sw = reinterpret_cast<uint32_t*>(&su);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float x0 = acc[2 * i], x1 = acc[2 * i + 1];
        if (bias != nullptr) {
          x0 += __bfloat162float(bias[idx * 8 + 2 * i]);
          x1 += __bfloat162float(bias[idx * 8 + 2 * i + 1]);
        }
        // same rounding points as GEMM -> bf16, then bf16 add
        x0 = __bfloat162float(__float2bfloat16(x0));
        x1 = __bfloat162float(__float2bfloat16(x1));
        const float2 r = __bfloat1622float2(rh[i]);
        sw[i] = pack_bf16(x0 + r.x, x1 + r.y);
      }
      *rp = su;
      const __nv_bfloat162* sh = reinterpret_cast<const __nv_bfloat162*>(&su);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(sh[i]);
        v[c][2 * i] = f.x;
        v[c][2 * i + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
      }
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < PN_THREADS / 32; ++i) tot += red[i];
  const float inv = rsqrtf(tot / float(H) + eps);
#pragma unroll
  for (int c = 0; c < PN_MAX_CHUNKS; ++c) {
    const int idx = threadIdx.x + c * PN_THREADS;
    if (idx < chunks) {
      const uint4 gu = *reinterpret_cast<const uint4*>(w + idx * 8);
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gu);
      uint4 ou;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&ou);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 g2 = __bfloat1622float2(gh[i]);
        ow[i] = pack_bf16(__bfloat162float(__float2bfloat16(v[c][2 * i] * inv)) * g2.x,
                          __bfloat162float(__float2bfloat16(v[c][2 * i + 1] * inv)) * g2.y);
      }
      *reinterpret_cast<uint4*>(y + row * H + idx * 8) = ou;
    }
  }
}

// out[t, i] = silu(g) * u with g = sum_s partial[s, t, i], u = sum_s partial[s, t, I + i]
__global__ void silu_mul_partials_kernel(const float* __restrict__ partial, int splits, long long split_stride,
                                         bf16* __restrict__ out, long long T, int I) {
  pdl_launch_dependents();
  pdl_wait();
  const int quads = I >> 2;
  const long long total = T * quads;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / quads;
    const int c = int(idx - t * quads) * 4;
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
    const float* base = partial + t * 2 * I + c;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
      const float4 a = __ldcg(reinterpret_cast<const float4*>(base + s * split_stride));
      const float4 b = __ldcg(reinterpret_cast<const float4*>(base + s * split_stride + I));
      g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
      u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
    }
    auto f = [](float gg, float uu) {
      gg = __bfloat162float(__float2bfloat16(gg));
      uu = __bfloat162float(__float2bfloat16(uu));
      return gg / (1.f + __expf(-gg)) * uu;
    };
    uint2 o;
    o.x = pack_bf16(f(g.x, u.x), f(g.y, u.y));
    o.y = pack_bf16(f(g.z, u.z), f(g.w, u.w));
    *reinterpret_cast<uint2*>(out + t * I + c) = o;
  }
}

void launch_add_rms_norm_partials(const float* partial, int splits, long long split_stride, const void* bias,
                                  void* residual, const void* w, void* y, long long T, int H, float eps,
                                  cudaStream_t s) {
  if (T == 0) return;
  launch_pdl(PDL_PARTIALS, add_rms_norm_partials_kernel, dim3((unsigned)T), dim3(PN_THREADS), 0, s, partial, splits, split_stride,
             (const bf16*)bias, (bf16*)residual, (const bf16*)w, (bf16*)y, H, eps);
}

void launch_silu_mul_partials(const float* partial, int splits, long long split_stride, void* out, long long T,
                              int I, cudaStream_t s) {
  if (T == 0) return;
  const long long total = T * (I >> 2);
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148 * 8);
  launch_pdl(PDL_PARTIALS, silu_mul_partials_kernel, dim3(blocks), dim3(256), 0, s, partial, splits, split_stride, (bf16*)out, T, I);
}

}  // namespace fc
