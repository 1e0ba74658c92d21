// bf16 GEMM for prefill sizes on CTA pairs: D[i, j] = act(sum_k A[i, k] * B[j, k] + bias[j]), tokens on the row
// operand, 256 x 256 output tile per pair of CTAs (a thread-block cluster of two, one CTA per SM).
//
// With one CTA per 128 x 256 tile (gemm.cu) every SM copies a whole 256 x 64 B tile per K block into its shared
// memory and its tensor core reads all of it back: shared-memory traffic, not the tensor pipe, bounds that kernel
// (81 % tensor-pipe activity).  Here the two CTAs of a pair issue ONE tcgen05.mma.cta_group::2 of M = 256, N = 256:
// each CTA holds 128 rows of A and 128 of the 256 rows of B, the tensor cores exchange the B halves between the
// two SMs, and each CTA's tensor memory receives its 128 x 256 half of the accumulator.  Per FLOP a CTA copies and
// reads two thirds of the operand bytes, and six pipeline stages fit where four did.
//
//   warp 0   TMA producer in BOTH CTAs: its own A tile and B half per stage (plain 2-D tiled loads from this
//            GPU's memory; every CTA fetches its own tiles), completion counted on the LEADER's (rank 0) barrier
//   warp 1   leader only: tcgen05.mma.cta_group::2 (4 x K = 16 per stage); tcgen05.commit to both CTAs' barriers
//            frees the stage in both and publishes the accumulator to both epilogues
//   warps 2-5 epilogue in both CTAs: tcgen05.ld of the CTA's own 128 x 256 fp32 half, bias / activation / SwiGLU,
//            16-byte bf16 stores; the 256 epilogue threads of the pair hand the accumulator back to the leader
// Two accumulators (2 x 256 TMEM columns per CTA) let the epilogue overlap the next tile's main loop.
//
// Every wait is bounded; both CTAs always reach the closing cluster barrier, so neither exits while its partner
// may still signal one of its barriers.
//
// Measured (32768 x 6144 x 4096): tensor pipe 88.5 % active against 81.1 % for gemm.cu, but both kernels run into
// the board's power limit (SM clock about 1.44 GHz) and take the same time within noise, so gemm_bf16 uses this
// kernel only when asked to (FC_GEMM_PAIRS=1 / set_gemm_pairs(1)).  Asking for tiles 16 K blocks ahead to be
// brought into L2 (cp.async.bulk.prefetch.tensor) made the K = 12288 shape 30 % slower and was taken out.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <stdexcept>
#include <string>

#include "gemm.h"
#include "ptx.cuh"

namespace fc {

namespace {

constexpr int P2_BM = 128;          // rows of A per CTA (256 per pair)
constexpr int P2_BNH = 128;         // rows of B per CTA (256 per pair)
constexpr int P2_BN = 256;
constexpr int P2_BK = 64;
constexpr int P2_STAGES = 6;
constexpr int P2_THREADS = 192;
constexpr int P2_A_BYTES = P2_BM * P2_BK * 2;
constexpr int P2_B_BYTES = P2_BNH * P2_BK * 2;
constexpr int P2_STAGE_BYTES = P2_A_BYTES + P2_B_BYTES;              // 32 KiB per CTA
constexpr int P2_BAR_OFF = P2_STAGES * P2_STAGE_BYTES;
constexpr int P2_SMEM = P2_BAR_OFF + 256 + 1024;

struct Pair2Params {
  int M, N, K;
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* bias;
  int act;
  int num_m, num_n, group_m, total_work;
  int up_row0;            // SWIGLU: row of W where the `up` half starts (= output width)
  uint32_t* status;
};

__device__ __forceinline__ float p2_act(float v, int act) {
  switch (act) {
    case ACT_RELU: return fmaxf(v, 0.f);
    case ACT_GELU: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    case ACT_GELU_TANH: {
      float u = 0.7978845608028654f * (v + 0.044715f * v * v * v), th;
      asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(u));
      return 0.5f * v * (1.f + th);
    }
    case ACT_QUICK_GELU: return __fdividef(v, 1.f + __expf(-1.702f * v));
    case ACT_SILU: return __fdividef(v, 1.f + __expf(-v));
    default: return v;
  }
}

// 2-D tiled load whose completion is counted on a barrier of the pair's leader CTA (`bar_cluster_addr` is a
// shared::cluster address); the destination is this CTA's own shared memory
__device__ __forceinline__ void p2_tma_load(void* smem, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void p2_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives (once the MMAs issued so far are done) on the barrier at this shared-memory offset in both CTAs
__device__ __forceinline__ void p2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}
__device__ __forceinline__ void p2_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

template <bool SWIGLU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P2_THREADS, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const Pair2Params p) {
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared memory starts at the same offset in both CTAs, so the aligned base does too
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + P2_BAR_OFF);      // used in the leader
  uint64_t* empty_bar = full_bar + P2_STAGES;                               // one set per CTA
  uint64_t* acc_full = empty_bar + P2_STAGES;                               // [2], one set per CTA
  uint64_t* acc_empty = acc_full + 2;                                       // [2], used in the leader (256 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P2_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 256);
    }
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    // all 512 columns in each CTA: both allocations start at column 0, which the pair's MMA relies on
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  cluster_sync();                                   // the partner's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_kb = (p.K + P2_BK - 1) / P2_BK;

  auto decode_work = [&](int w, int& m_blk, int& n_blk) {
    const int per_group = p.group_m * p.num_n;
    const int g = w / per_group;
    const int first_m = g * p.group_m;
    const int gm = min(p.num_m - first_m, p.group_m);
    const int local = w - g * per_group;
    m_blk = first_m + local % gm;
    n_blk = local / gm;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = tmem_base == 0;
      if (!ok) report(p.status, ST_BAD_INDEX);      // the allocation did not start at column 0: do not run
      for (int w = pair; w < p.total_work && ok; w += num_pairs) {
        int m_blk, n_blk;
        decode_work(w, m_blk, n_blk);
        const int a_row = m_blk * (2 * P2_BM) + int(rank) * P2_BM;
        const int b_row = SWIGLU ? (rank == 0 ? n_blk * P2_BNH : p.up_row0 + n_blk * P2_BNH)
                                 : n_blk * P2_BN + int(rank) * P2_BNH;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (*s_abort || !mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_EMPTY)) {
            *s_abort = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * P2_STAGE_BYTES;
          const uint32_t bar = cluster_map_shared(smem_u32(&full_bar[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * P2_STAGE_BYTES);      // both CTAs' bytes
          p2_tma_load(sa, &tma_a, bar, kb * P2_BK, a_row);
          p2_tma_load(sa + P2_A_BYTES, &tma_b, bar, kb * P2_BK, b_row);
          if (++stage == P2_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (ok) {
        // the leader's last commits also arrive on this CTA's stage barriers: let them land before the closing
        // cluster barrier (an unused stage passes at once)
        for (int n = 0; n < P2_STAGES; ++n) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_EMPTY)) break;
          if (++stage == P2_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      } else {
        // gave up: a copy requested just before may still be on its way into this CTA's shared memory
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && rank == 0 && tmem_base == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * P2_BM, P2_BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int w = pair; w < p.total_work && ok; w += num_pairs) {
        if (*s_abort || !mbar_wait(&acc_empty[acc], acc_phase ^ 1, p.status, ST_TIMEOUT_ACC_EMPTY)) {
          *s_abort = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(acc * P2_BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (*s_abort || !mbar_wait(&full_bar[stage], phase, p.status, ST_TIMEOUT_FULL)) {
            *s_abort = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * P2_STAGE_BYTES);
          const uint64_t da = make_sdesc_sw128(sa);
          const uint64_t db = make_sdesc_sw128(sa + P2_A_BYTES);
#pragma unroll
          for (int k = 0; k < P2_BK / 16; ++k)
            p2_mma(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          p2_commit_both(&empty_bar[stage]);
          if (++stage == P2_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        p2_commit_both(&acc_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs)
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int w = pair; w < p.total_work; w += num_pairs) {
      int m_blk, n_blk;
      decode_work(w, m_blk, n_blk);
      if (*s_abort || !mbar_wait(&acc_full[acc], acc_phase, p.status, ST_TIMEOUT_ACC_FULL)) {
        *s_abort = 1;
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (uint32_t(lane_group * 32) << 16) + uint32_t(acc * P2_BN);
      const uint32_t give_back = cluster_map_shared(smem_u32(&acc_empty[acc]), 0);
      const int gi = m_blk * (2 * P2_BM) + int(rank) * P2_BM + row;
      if constexpr (SWIGLU) {
        // accumulator columns [0, 128) = gate, [128, 256) = up; out[:, n_blk * 128 + j] = silu(gate_j) * up_j
        const int jo = n_blk * P2_BNH;
#pragma unroll 1
        for (int c = 0; c < P2_BNH / 32; ++c) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(t_addr + uint32_t(c * 32), rg);
          tmem_ld_32x32(t_addr + uint32_t(P2_BNH + c * 32), ru);
          tmem_ld_wait();
          if (c == P2_BNH / 32 - 1) {
            tc_fence_before();
            p2_arrive_cluster(give_back);
          }
          if (gi < p.M) {
            __nv_bfloat16* dst = p.C + (long long)gi * p.ldc + jo + c * 32;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t u[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int t = q * 8 + e * 2;
                const float g0 = __uint_as_float(rg[t]), g1 = __uint_as_float(rg[t + 1]);
                const float a = __fdividef(g0, 1.f + __expf(-g0)) * __uint_as_float(ru[t]);
                const float b = __fdividef(g1, 1.f + __expf(-g1)) * __uint_as_float(ru[t + 1]);
                u[e] = pack_bf16(a, b);
              }
              *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(u[0], u[1], u[2], u[3]);
            }
          }
        }
      } else {
        const int j0 = n_blk * P2_BN;
#pragma unroll 1
        for (int c = 0; c < P2_BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_addr + uint32_t(c * 32), r);
          tmem_ld_wait();
          if (c == P2_BN / 32 - 1) {
            tc_fence_before();
            p2_arrive_cluster(give_back);
          }
          const int jb = j0 + c * 32;
          if (gi >= p.M || jb >= p.N) continue;
          float v[32];
#pragma unroll
          for (int t = 0; t < 32; ++t) v[t] = __uint_as_float(r[t]);
          __nv_bfloat16* dst = p.C + (long long)gi * p.ldc + jb;
          const bool vec_ok = (jb + 32 <= p.N) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
          if (vec_ok) {
            if (p.bias != nullptr) {
              if ((reinterpret_cast<uintptr_t>(p.bias + jb) & 15) == 0) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + jb + q * 8);
                  const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {      // a bf16 is the upper half of the fp32 with the same value
                    v[q * 8 + e * 2] += __uint_as_float(bw[e] << 16);
                    v[q * 8 + e * 2 + 1] += __uint_as_float(bw[e] & 0xffff0000u);
                  }
                }
              } else {
#pragma unroll
                for (int t = 0; t < 32; ++t) v[t] += __bfloat162float(p.bias[jb + t]);
              }
            }
            if (p.act != ACT_NONE) {
#pragma unroll
              for (int t = 0; t < 32; ++t) v[t] = p2_act(v[t], p.act);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t u[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) u[e] = pack_bf16(v[q * 8 + e * 2], v[q * 8 + e * 2 + 1]);
              *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(u[0], u[1], u[2], u[3]);
            }
          } else {
#pragma unroll
            for (int t = 0; t < 32; ++t) {
              if (jb + t < p.N) {
                float a = v[t];
                if (p.bias != nullptr) a += __bfloat162float(p.bias[jb + t]);
                dst[t] = __float2bfloat16(p2_act(a, p.act));
              }
            }
          }
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  tc_fence_before();
  cluster_sync();                                   // nothing of the partner's is signalled after this
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

int g_pairs = -1;

template <bool SWIGLU>
void p2_launch(const CUtensorMap& ta, const CUtensorMap& tb, const Pair2Params& p, int pairs, cudaStream_t stream) {
  auto kern = gemm_bf16_2cta_kernel<SWIGLU>;
  static std::atomic<uint64_t> configured{0};
  int dev = 0;
  cudaGetDevice(&dev);
  const uint64_t bit = 1ull << (dev & 63);
  if (!(configured.load(std::memory_order_relaxed) & bit)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P2_SMEM);
    if (e != cudaSuccess) throw std::runtime_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    configured.fetch_or(bit, std::memory_order_relaxed);
  }
  kern<<<2 * pairs, P2_THREADS, P2_SMEM, stream>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("2-CTA gemm launch: ") + cudaGetErrorString(e));
}

}  // namespace

int gemm_pairs_mode() {
  if (g_pairs < 0) {
    const char* e = std::getenv("FC_GEMM_PAIRS");
    g_pairs = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  return g_pairs;
}
void set_gemm_pairs(int mode) { g_pairs = mode ? 1 : 0; }

bool gemm_bf16_2cta(const void* x, const void* w, void* c, const void* bias, int M, int N, int K, long long ldx,
                    long long ldw, long long ldc, int act, int sm_limit, uint32_t* status, cudaStream_t stream) {
  const bool swiglu = act == ACT_SWIGLU;
  if (M <= 256 || N < 256 || K < P2_BK) return false;
  if (swiglu && (N % 256 != 0 || ldc % 8 != 0 || (reinterpret_cast<uintptr_t>(c) & 15) != 0 || bias != nullptr))
    return false;
  const int sms = sm_limit > 0 ? sm_limit : gemm_num_sms();
  if (sms < 2) return false;
  Pair2Params p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.C = reinterpret_cast<__nv_bfloat16*>(c);
  p.ldc = ldc;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.act = swiglu ? ACT_NONE : act;
  p.num_m = (M + 2 * P2_BM - 1) / (2 * P2_BM);
  p.num_n = swiglu ? N / 256 : (N + P2_BN - 1) / P2_BN;
  // raster: groups of `group_m` row blocks are finished one after the other, all column blocks of one before the
  // next.  The group's rows of A (group_m x 256 x K) stay in L2 while B streams past once per group, so larger groups
  // mean fewer passes over B; about 32 MB of A is what stays resident beside the streams (the L2 is two 63 MB halves).
  {
    const char* e = std::getenv("FC_GEMM_GROUP_M");
    const long long a_block = 2ll * 256 * K;
    p.group_m = e != nullptr ? std::max(1, std::atoi(e)) : int(std::max(8ll, std::min(32ll, (32ll << 20) / a_block)));
  }
  p.total_work = p.num_m * p.num_n;
  p.up_row0 = N / 2;
  p.status = status;
  const CUtensorMap ta = make_tmap_bf16_2d(x, M, K, ldx, P2_BM, P2_BK);
  const CUtensorMap tb = make_tmap_bf16_2d(w, N, K, ldw, P2_BNH, P2_BK);
  const int pairs = std::max(1, std::min(p.total_work, sms / 2));
  if (swiglu) p2_launch<true>(ta, tb, p, pairs, stream);
  else p2_launch<false>(ta, tb, p, pairs, stream);
  return true;
}

}  // namespace fc
