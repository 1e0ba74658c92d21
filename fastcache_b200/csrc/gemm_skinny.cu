// Weight-streaming GEMM for decode-size batches (M <= 256 tokens): y[M, N] = x[M, K] @ W[N, K]^T.
//
// At these sizes the op is bound by reading W from HBM once.  The weight matrix is
// therefore the 128-row tcgen05 operand ("swapped" form) and the token batch is the
// N operand, so one CTA covers *all* tokens for its rows of W and W is never read
// twice.  A CTA owns 256 rows of W (two M = 128 MMAs that share one x tile in shared
// memory, which halves the re-reads of x from L2) and a slice of K:
//
//   grid = (N / 256 tiles) x (K splits), chosen so the CTA count is close to a
//   multiple of the SM count
//   warp 0: TMA producer (W tile 256 x 64 and x tile BN x 64 per stage, 128-byte swizzle)
//   warp 1: tcgen05.mma issuer, accumulators in TMEM (2 x BN fp32 columns)
//   warps 2-5: epilogue, tcgen05.ld -> transposed store
//
// With one split the epilogue writes bf16 (bias and activation applied).  With
// several it writes fp32 partial sums [split, M, N] to scratch; the partials are
// summed by the kernel that consumes the result (add + RMSNorm and SwiGLU in
// partials.cu, rope + KV store in elementwise.cu, the one-shot all-reduce in comm.cu)
// or by the small finalize kernel below.  No inter-CTA synchronisation is needed.
//
// Fused epilogues (row-parallel projections o_proj / down_proj of a decode step): with `epi` set the kernel
// goes on after its partial sums are written.  All CTAs meet at a grid barrier (the grid never exceeds the SM
// count, one CTA per SM, so all of them are resident), then every CTA takes token rows c, c + grid, ...:
//   EPI_ADD_NORM     sum of the split-K partials (+ bias) + residual -> residual, RMSNorm -> y
//   EPI_AR_ADD_NORM  the same with the sum over tensor-parallel ranks in between: the CTA finishes its rows into
//                    this rank's symmetric staging buffer, exchanges flags with the same CTA of every peer and
//                    reads the peers' rows (plain peer loads in rank order, or multimem.ld_reduce)
// which replaces the GEMM -> (all-reduce +) add + RMSNorm pair of launches by one.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <stdexcept>
#include <string>

#include "comm.h"
#include "comm_dev.cuh"
#include "gemm.h"
#include "launch.h"
#include "ptx.cuh"

namespace fc {

constexpr int SK_BM = 256;       // rows of W per CTA
constexpr int SK_BK = 64;
constexpr int SK_THREADS = 192;

struct SkinnyParams {
  int Nw;                 // rows of W (output features)
  int Mtok;               // tokens
  int K;
  __nv_bfloat16* out;     // [Mtok, ldc] bf16 (splits == 1)
  long long ldc;
  float* partial;         // [splits, Mtok, Nw] fp32 (splits > 1)
  const __nv_bfloat16* bias;
  int act;
  int splits;
  int kb_per_split;
  uint32_t* status;
  // fused epilogue (see the header comment); epi == EPI_NONE: everything below is unused
  int epi;
  uint32_t* grid_sync;            // [0] arrivals, [1] generation
  __nv_bfloat16* residual;        // [Mtok, Nw], updated in place
  const __nv_bfloat16* norm_w;    // [Nw]
  __nv_bfloat16* y;               // [Mtok, Nw]
  float eps;
  CommPeers peers;                // EPI_AR_ADD_NORM
  int buf;
  const __nv_bfloat16* mc_in;     // multicast address of staging buffer `buf`, or nullptr for peer loads
  uint32_t* epochs;
};

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }   // the 4 epilogue warps

// Grid barrier for the 128 epilogue threads of every CTA (tid = 0..127).  Sense reversal: the generation word is
// read before arriving (it cannot move until this CTA has arrived too), the last arriver resets the count and
// bumps the generation, so the two words are ready for the next launch (also a replay from a CUDA graph).
// Returns false when the bounded wait ran out.
__device__ __forceinline__ bool skinny_grid_barrier(const SkinnyParams& p, int tid, int nctas, volatile int* s_flag) {
  __threadfence();                         // this thread's partial sums, before the arrival
  epi_bar();
  if (tid == 0) {
    volatile uint32_t* gen_p = p.grid_sync + 1;
    const uint32_t gen = *gen_p;
    __threadfence();
    bool ok = true;
    if (atomicAdd(p.grid_sync, 1u) == uint32_t(nctas - 1)) {
      *reinterpret_cast<volatile uint32_t*>(p.grid_sync) = 0u;
      __threadfence();
      atomicAdd(p.grid_sync + 1, 1u);
    } else {
      const uint64_t t0 = global_timer_ns();
      uint64_t limit = FC_WAIT_LIMIT_NS;
      ok = false;
      for (uint32_t i = 0; i < (1u << 28); ++i) {
        if (*gen_p != gen) {
          ok = true;
          break;
        }
        if ((i & 255u) == 255u) {
          if (i == 255u) limit = status_wait_limit_ns(p.status, FC_WAIT_LIMIT_NS);
          if (global_timer_ns() - t0 > limit) break;
        }
      }
      if (!ok) report(p.status, ST_TIMEOUT_GRID);
    }
    __threadfence();
    *s_flag = ok ? 1 : 0;
  }
  epi_bar();
  return *s_flag != 0;
}

constexpr int EPI_MAX_CHUNKS = 8;          // 16-byte pieces per thread and row: hidden <= 128 * 8 * 8 = 8192

// sum over the K splits of 8 consecutive outputs of one token row (+ bias)
__device__ __forceinline__ void skinny_sum_splits(const SkinnyParams& p, long long off, int col, float (&acc)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  const long long stride = (long long)p.Mtok * p.Nw;
#pragma unroll 4
  for (int s = 0; s < p.splits; ++s) {
    const float4* ps = reinterpret_cast<const float4*>(p.partial + s * stride + off);
    const float4 a = __ldcg(ps), b = __ldcg(ps + 1);
    acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
    acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
  }
  if (p.bias != nullptr) {
    float bb[8];
    unpack8f(*reinterpret_cast<const uint4*>(p.bias + col), bb);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += bb[i];
  }
}

// The row phase of the fused epilogues, run by the 128 epilogue threads of CTA `cta` of `nctas`.
__device__ __noinline__ void skinny_row_phase(const SkinnyParams& p, int cta, int nctas, int tid, float* s_red,
                                              volatile int* s_flag, uint32_t* s_epoch) {
  const int H = p.Nw;
  const int chunks = H >> 3;
  if (p.epi == EPI_AR_ADD_NORM) {
    // this rank's contribution of my rows -> staging buffer (bf16, the rounding point of a GEMM output)
    __nv_bfloat16* mine = p.peers.data[p.buf][p.peers.rank];
    for (int row = cta; row < p.Mtok; row += nctas) {
      for (int idx = tid; idx < chunks; idx += 128) {
        const long long off = (long long)row * H + (long long)idx * 8;
        float acc[8];
        skinny_sum_splits(p, off, idx * 8, acc);
        *reinterpret_cast<uint4*>(mine + off) = pack8f(acc);
      }
    }
    if (tid == 0) {
      *s_epoch = p.epochs[cta] + 1;
      *s_flag = 1;
    }
    epi_bar();                             // all rows of this CTA are written before any flag goes out
    const uint32_t epoch = *s_epoch;
    if (tid < p.peers.world && !peer_flag_exchange(p.peers, cta, epoch, tid, p.status)) *s_flag = 0;
    epi_bar();
    if (tid == 0) p.epochs[cta] = epoch;
    if (*s_flag == 0) return;              // the host reads the status word and raises
  }
  for (int row = cta; row < p.Mtok; row += nctas) {
    const long long base = (long long)row * H;
    float v[EPI_MAX_CHUNKS][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < EPI_MAX_CHUNKS; ++c) {
      const int idx = tid + c * 128;
      if (idx < chunks) {
        const long long off = base + (long long)idx * 8;
        float acc[8];
        if (p.epi == EPI_AR_ADD_NORM) {
          if (p.mc_in != nullptr) {
            unpack8f(multimem_ld_reduce_bf16x8(p.mc_in + off), acc);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0.f;
            uint4 raw[COMM_MAX_WORLD];     // every peer's piece is requested before the first is used
#pragma unroll
            for (int q = 0; q < COMM_MAX_WORLD; ++q)
              if (q < p.peers.world) raw[q] = ld_peer_16(p.peers.data[p.buf][q] + off);
#pragma unroll
            for (int q = 0; q < COMM_MAX_WORLD; ++q) {
              if (q < p.peers.world) {
                float f[8];
                unpack8f(raw[q], f);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += f[i];
              }
            }
          }
        } else {
          skinny_sum_splits(p, off, idx * 8, acc);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = __bfloat162float(__float2bfloat16(acc[i]));   // GEMM output rounding
        }
        float r[8];
        unpack8f(*reinterpret_cast<const uint4*>(p.residual + off), r);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += r[i];
        const uint4 sres = pack8f(acc);
        *reinterpret_cast<uint4*>(p.residual + off) = sres;
        unpack8f(sres, v[c]);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[c][i] * v[c][i];
      }
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) s_red[tid >> 5] = ss;
    epi_bar();
    const float tot = s_red[0] + s_red[1] + s_red[2] + s_red[3];
    epi_bar();
    const float inv = rsqrtf(tot / float(H) + p.eps);
#pragma unroll
    for (int c = 0; c < EPI_MAX_CHUNKS; ++c) {
      const int idx = tid + c * 128;
      if (idx < chunks) {
        float g[8], o[8];
        unpack8f(*reinterpret_cast<const uint4*>(p.norm_w + (size_t)idx * 8), g);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __bfloat162float(__float2bfloat16(v[c][i] * inv)) * g[i];
        *reinterpret_cast<uint4*>(p.y + base + (long long)idx * 8) = pack8f(o);
      }
    }
  }
}

__device__ __forceinline__ float sk_act(float v, int act) {
  switch (act) {
    case ACT_RELU: return fmaxf(v, 0.f);
    case ACT_GELU: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    case ACT_GELU_TANH: {
      float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
      return 0.5f * v * (1.f + tanhf(u));
    }
    case ACT_QUICK_GELU: return v / (1.f + __expf(-1.702f * v));
    case ACT_SILU: return v / (1.f + __expf(-v));
    default: return v;
  }
}

// ROWS = rows of W per CTA: 256 (two MMAs share the x tile) or 128 (twice the CTAs, for matrices with so few
// rows that 256-row tiles would leave most SMs without work, e.g. the per-rank shards under tensor parallelism)
template <int BN, int STAGES, int ROWS = SK_BM>
struct SkinnySmem {
  static constexpr int A_BYTES = ROWS * SK_BK * 2;
  static constexpr int B_BYTES = BN * SK_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFF = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

template <int BN, int STAGES, int ROWS>
__global__ void __launch_bounds__(SK_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x,
                   const SkinnyParams p) {
  using L = SkinnySmem<BN, STAGES, ROWS>;
  constexpr int MT = ROWS / 128;            // 128-row MMAs per K step
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* s_flag = s_abort + 1;                                   // fused epilogues
  uint32_t* s_epoch = reinterpret_cast<uint32_t*>(const_cast<int*>(s_abort + 2));
  float* s_red = reinterpret_cast<float*>(const_cast<int*>(s_abort + 4));   // 4 floats

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = (MT * BN <= 32) ? 32 : (MT * BN <= 64) ? 64 : (MT * BN <= 128) ? 128
                                 : (MT * BN <= 256) ? 256 : 512;
  const int tile = blockIdx.x, split = blockIdx.y;
  const int num_kb = (p.K + SK_BK - 1) / SK_BK;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(num_kb, kb0 + p.kb_per_split);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tma_w);
    tma_prefetch_desc(&tma_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool is_producer = (warp == 0 && lane == 0);
  if (!is_producer) {
    pdl_wait();                            // x, the scratch and the output belong to earlier kernels until here
  }

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      // The weights never change during serving: their first tiles are requested while the previous kernel
      // of the stream is still draining (programmatic dependent launch); only the activations wait for it.
      const int npre = min(STAGES, kb1 - kb0);
      for (int s = 0; s < npre; ++s) {
        uint8_t* sa = smem + s * L::STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
        tma_load_2d(sa, &tma_w, &full_bar[s], (kb0 + s) * SK_BK, tile * ROWS);
        if constexpr (MT == 2)
          tma_load_2d(sa + L::A_BYTES / 2, &tma_w, &full_bar[s], (kb0 + s) * SK_BK, tile * ROWS + 128);
      }
      pdl_wait();
      asm volatile("fence.proxy.async.global;" ::: "memory");   // x: ordinary stores before, TMA reads now
      for (int s = 0; s < npre; ++s)
        tma_load_2d(smem + s * L::STAGE_BYTES + L::A_BYTES, &tma_x, &full_bar[s], (kb0 + s) * SK_BK, 0);
      issued = npre;
      stage = npre == STAGES ? 0 : npre;
      phase = npre == STAGES ? 1u : 0u;
      for (int kb = kb0 + npre; kb < kb1; ++kb) {
        if (*s_abort || !mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_EMPTY)) {
          *s_abort = 1;
          ok = false;
          break;
        }
        uint8_t* sa = smem + stage * L::STAGE_BYTES;
        uint8_t* sb = sa + L::A_BYTES;
        mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
        tma_load_2d(sa, &tma_w, &full_bar[stage], kb * SK_BK, tile * ROWS);
        if constexpr (MT == 2)
          tma_load_2d(sa + L::A_BYTES / 2, &tma_w, &full_bar[stage], kb * SK_BK, tile * ROWS + 128);
        tma_load_2d(sb, &tma_x, &full_bar[stage], kb * SK_BK, 0);
        ++issued;
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) {
        int s = stage;
        uint32_t ph = phase;
        for (int n = 0; n < min(issued, STAGES); ++n) {
          if (--s < 0) {
            s = STAGES - 1;
            ph ^= 1;
          }
          mbar_wait(&full_bar[s], ph, nullptr, 0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (*s_abort || !mbar_wait(&full_bar[stage], phase, p.status, ST_TIMEOUT_FULL)) {
          *s_abort = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
        const uint64_t da0 = make_sdesc_sw128(sa);
        const uint64_t da1 = make_sdesc_sw128(sa + L::A_BYTES / 2);
        const uint64_t db = make_sdesc_sw128(sa + L::A_BYTES);
#pragma unroll
        for (int k = 0; k < SK_BK / 16; ++k) {
          const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
          tc_mma_f16(tmem_base, da0 + uint64_t(2 * k), db + uint64_t(2 * k), idesc, accum);
          if constexpr (MT == 2)
            tc_mma_f16(tmem_base + BN, da1 + uint64_t(2 * k), db + uint64_t(2 * k), idesc, accum);
        }
        tc_commit(&empty_bar[stage]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) tc_commit(acc_full);
    }
  } else {
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;
    const bool direct = p.splits == 1 && p.epi == EPI_NONE;     // bf16 result straight from the accumulator
    if (!*s_abort && mbar_wait(acc_full, 0, p.status, ST_TIMEOUT_ACC_FULL)) {
      tc_fence_after();
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        const int n = tile * ROWS + mt * 128 + row;           // output feature of this thread
        const uint32_t t_addr = tmem_base + (uint32_t(lane_group * 32) << 16) + uint32_t(mt * BN);
        const float bi = (p.bias != nullptr && n < p.Nw && direct) ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_addr + uint32_t(c * 32), r);
          tmem_ld_wait();
          if (n < p.Nw) {
            if (direct) {
#pragma unroll
              for (int t = 0; t < 32; ++t) {
                const int tok = c * 32 + t;
                if (tok < p.Mtok)
                  p.out[(long long)tok * p.ldc + n] = __float2bfloat16(sk_act(__uint_as_float(r[t]) + bi, p.act));
              }
            } else {
              float* dst = p.partial + ((long long)split * p.Mtok) * p.Nw + n;
#pragma unroll
              for (int t = 0; t < 32; ++t) {
                const int tok = c * 32 + t;
                if (tok < p.Mtok) dst[(long long)tok * p.Nw] = __uint_as_float(r[t]);
              }
            }
          }
        }
      }
    }
    if (p.epi != EPI_NONE) {
      // every CTA joins the barrier, also one whose pipeline gave up (its partial sums are then missing and the
      // status word says so): the others must not wait for it until their own limit
      const int nctas = gridDim.x * gridDim.y;
      const int cta = blockIdx.y * gridDim.x + blockIdx.x;
      const int etid = (warp - 2) * 32 + lane;
      if (skinny_grid_barrier(p, etid, nctas, s_flag))
        skinny_row_phase(p, cta, nctas, etid, s_red, s_flag, s_epoch);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// out[m, n] = act(sum_s partial[s, m, n] + bias[n])
__global__ void skinny_finalize_kernel(const float* __restrict__ partial, const __nv_bfloat16* __restrict__ bias,
                                       __nv_bfloat16* __restrict__ out, int M, int N, long long ldc, int splits,
                                       int act) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)M * (N / 4);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int m = int(i / (N / 4)), n = int(i % (N / 4)) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(partial + ((long long)s * M + m) * N + n);
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    if (bias != nullptr) {
      acc.x += __bfloat162float(bias[n]);
      acc.y += __bfloat162float(bias[n + 1]);
      acc.z += __bfloat162float(bias[n + 2]);
      acc.w += __bfloat162float(bias[n + 3]);
    }
    __nv_bfloat16* o = out + (long long)m * ldc + n;
    o[0] = __float2bfloat16(sk_act(acc.x, act));
    o[1] = __float2bfloat16(sk_act(acc.y, act));
    o[2] = __float2bfloat16(sk_act(acc.z, act));
    o[3] = __float2bfloat16(sk_act(acc.w, act));
  }
}

template <int BN, int STAGES, int ROWS>
static void launch_skinny(const CUtensorMap& tw, const CUtensorMap& tx, const SkinnyParams& p, int tiles,
                          cudaStream_t stream) {
  using L = SkinnySmem<BN, STAGES, ROWS>;
  auto kern = gemm_skinny_kernel<BN, STAGES, ROWS>;
  // the attribute belongs to the (function, device) pair: remember it per device, not per process
  static std::atomic<uint64_t> configured{0};
  int dev = 0;
  cudaGetDevice(&dev);
  const uint64_t bit = 1ull << (dev & 63);
  if (!(configured.load(std::memory_order_relaxed) & bit)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) throw std::runtime_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    configured.fetch_or(bit, std::memory_order_relaxed);
  }
  cudaError_t e = launch_pdl(PDL_SKINNY_GEMM, kern, dim3(tiles, p.splits), dim3(SK_THREADS), L::TOTAL, stream, tw, tx, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("skinny gemm launch: ") + cudaGetErrorString(e));
}

// Number of K splits for `tiles` row tiles on `sms` SMs: fill the machine to a whole
// number of waves while keeping at least 4 K blocks per CTA.
int skinny_pick_splits(int tiles, int tile_rows, int num_kb, int sms, int M, int N, size_t scratch_floats,
                       int max_ctas = 1 << 30) {
  int best = 1;
  double best_cost = 1e30;
  const int max_s = std::max(1, std::min(num_kb / 4, 32));
  for (int s = 1; s <= max_s; ++s) {
    if (s > 1 && (size_t)s * M * N > scratch_floats) break;
    if (s > 1 && tiles * s > max_ctas) break;      // fused epilogues: the whole grid is resident at once
    const int ctas = tiles * s;
    const int waves = (ctas + sms - 1) / sms;
    const int kb = (num_kb + s - 1) / s;
    // time ~ waves * (kb + fixed overhead per CTA), in units of one k-block step of a full wave; partial traffic
    // adds a little per split while the fp32 partial sums stay in L2 (every extra split is another copy of the
    // output for the consumer to read back), and their full write + read-back once they no longer fit (the LM
    // head: 128 x 151936 x 4 bytes per split), counted against the weight bytes a wave moves per step
    double cost = waves * (kb + 6.0) + 0.5 * s;
    if (s > 1) {
      const double partial_bytes = 4.0 * s * M * N, l2_resident = 48.0 * 1024 * 1024;
      if (partial_bytes > l2_resident)
        cost += 2.0 * (partial_bytes - l2_resident) / (double(sms) * tile_rows * SK_BK * 2.0);
    }
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

// Returns the number of splits used.  splits_request: 0 = choose; when the result is > 1 and
// `finalize` is false the caller consumes ws.scratch as fp32 [splits, M, N] itself.
int gemm_skinny_bf16(const void* x, const void* w, void* c, const void* bias, int M, int N, int K, long long ldx,
                     long long ldw, long long ldc, int act, const GemmWorkspace& ws, int sm_limit,
                     int splits_request, bool finalize, cudaStream_t stream, const SkinnyFused* fused) {
  const int sms = sm_limit > 0 ? sm_limit : gemm_num_sms();
  const int num_kb = (K + SK_BK - 1) / SK_BK;
  // 128-row tiles when 256-row tiles would cover less than half of the SMs: the same SM count is then reached
  // with half the K splits, i.e. half the partial-sum traffic
  const bool small_rows = (N + SK_BM - 1) / SK_BM <= sms / 2;
  const int rows = small_rows ? 128 : SK_BM;
  const int tiles = (N + rows - 1) / rows;
  const size_t scratch_floats = ws.scratch != nullptr ? gemm_scratch_bytes() / 4 : 0;
  const bool fuse = fused != nullptr && fused->epi != EPI_NONE;
  if (fuse) {
    // the fused epilogues need the whole grid resident (one CTA per SM), partial sums for every split, and rows
    // of 16-byte pieces that 128 threads cover in EPI_MAX_CHUNKS steps
    if (tiles > sms || N % 8 != 0 || N > 128 * EPI_MAX_CHUNKS * 8 || ws.grid_sync == nullptr ||
        (size_t)M * N > scratch_floats)
      return 0;
  }
  int splits = splits_request > 0 ? splits_request
                                  : skinny_pick_splits(tiles, rows, num_kb, sms, M, N, scratch_floats, fuse ? sms : 1 << 30);
  if (N % 4 != 0) splits = 1;
  if (splits > 1 && (size_t)splits * M * N > scratch_floats) splits = 1;
  if (fuse && tiles * splits > sms) splits = std::max(1, sms / tiles);
  int kb_per = (num_kb + splits - 1) / splits;
  splits = (num_kb + kb_per - 1) / kb_per;
  SkinnyParams p{};
  p.Nw = N;
  p.Mtok = M;
  p.K = K;
  p.out = reinterpret_cast<__nv_bfloat16*>(c);
  p.ldc = ldc;
  p.partial = ws.scratch;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.act = act;
  p.splits = splits;
  p.kb_per_split = kb_per;
  p.status = ws.status;
  if (fuse) {
    p.epi = fused->epi;
    p.grid_sync = ws.grid_sync;
    p.residual = reinterpret_cast<__nv_bfloat16*>(fused->residual);
    p.norm_w = reinterpret_cast<const __nv_bfloat16*>(fused->norm_w);
    p.y = reinterpret_cast<__nv_bfloat16*>(fused->y);
    p.eps = fused->eps;
    if (fused->epi == EPI_AR_ADD_NORM) {
      if (fused->peers == nullptr || fused->epochs == nullptr || tiles * splits > COMM_MAX_SLOTS)
        throw std::runtime_error("fused all-reduce epilogue: communication state is missing");
      p.peers = *fused->peers;
      p.buf = fused->buf;
      p.mc_in = reinterpret_cast<const __nv_bfloat16*>(fused->mc_in);
      p.epochs = fused->epochs;
    }
  }
  CUtensorMap tw = make_tmap_bf16_2d(w, N, K, ldw, 128, SK_BK);
  if (M <= 32) {
    CUtensorMap tx = make_tmap_bf16_2d(x, M, K, ldx, 32, SK_BK);
    if (small_rows) launch_skinny<32, 8, 128>(tw, tx, p, tiles, stream);
    else launch_skinny<32, 6, 256>(tw, tx, p, tiles, stream);
  } else if (M <= 64) {
    CUtensorMap tx = make_tmap_bf16_2d(x, M, K, ldx, 64, SK_BK);
    if (small_rows) launch_skinny<64, 7, 128>(tw, tx, p, tiles, stream);
    else launch_skinny<64, 5, 256>(tw, tx, p, tiles, stream);
  } else if (M <= 128) {
    CUtensorMap tx = make_tmap_bf16_2d(x, M, K, ldx, 128, SK_BK);
    if (small_rows) launch_skinny<128, 6, 128>(tw, tx, p, tiles, stream);
    else launch_skinny<128, 4, 256>(tw, tx, p, tiles, stream);
  } else {
    CUtensorMap tx = make_tmap_bf16_2d(x, M, K, ldx, 256, SK_BK);
    if (small_rows) launch_skinny<256, 4, 128>(tw, tx, p, tiles, stream);
    else launch_skinny<256, 3, 256>(tw, tx, p, tiles, stream);
  }
  if (splits > 1 && finalize && !fuse) {
    const long long total = (long long)M * (N / 4);
    const int blocks = (int)std::min<long long>((total + 255) / 256, 2048);
    launch_pdl(PDL_FINALIZE, skinny_finalize_kernel, dim3(blocks), dim3(256), 0, stream, (const float*)ws.scratch, p.bias, p.out, M,
               N, ldc, splits, act);
  }
  return splits;
}

}  // namespace fc
