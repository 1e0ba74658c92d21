// bf16 GEMM for sm_100a: D[i, j] = act(sum_k A[i, k] * B[j, k] + bias), fp32 accumulation in TMEM.
//
// Both operands are K-major ("TN"), which is what activations [tokens, K] and
// nn.Linear weights [out, K] are.  One persistent CTA per SM walks a list of
// (output tile, K split) work items:
//
//   warp 0   TMA producer: cp.async.bulk.tensor 2-D loads (128-byte swizzle) of a
//            128 x 64 A tile and a BN x 64 B tile per stage into a STAGES-deep ring
//   warp 1   MMA issuer: tcgen05.mma (cta_group::1, kind::f16, M = 128, N = BN,
//            K = 16) x 4 per stage; tcgen05.commit releases the stage and, after the
//            last K block, publishes the accumulator
//   warps 2-5 epilogue: tcgen05.ld of the 128 x BN fp32 accumulator (one TMEM lane
//            per thread), bias / activation, bf16 stores
// Two accumulators (2 x BN TMEM columns) let the epilogue of one tile overlap the
// main loop of the next.
//
// Output addressing is (i, j) -> C + i * ldc_i + j * ldc_j, so the same kernel
// serves the "swapped" decode form in which the weight matrix is the 128-row
// operand and the (small) token batch is the N operand: W is then streamed from
// HBM exactly once per step and the result is written transposed.
//
// Split-K (decode shapes with few output tiles): each split stores its fp32
// partial tile to scratch; a per-tile arrival counter elects the last split, which
// sums the partials in split order (deterministic), applies the epilogue and
// resets the counter.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>

#include "gemm.h"
#include "ptx.cuh"

namespace fc {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  int M, N, K;
  __nv_bfloat16* C;
  long long ldc_i, ldc_j;
  const __nv_bfloat16* bias;
  int bias_on_i;
  int act;
  int splits;
  int kb_per_split;
  float* scratch;
  int* counters;
  uint32_t* status;
  int num_m, num_n, group_m;
  int total_work;
  int up_row0;            // SWIGLU: row of W where the `up` half starts (= output width)
};

__device__ __forceinline__ float apply_act(float v, int act) {
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

// The activation of 32 values with the (uniform) selector tested once, not per element.
__device__ __forceinline__ void apply_act_chunk(float (&v)[32], int act) {
  switch (act) {
    case ACT_NONE: break;
    case ACT_RELU:
#pragma unroll
      for (int t = 0; t < 32; ++t) v[t] = apply_act(v[t], ACT_RELU);
      break;
    case ACT_GELU:
#pragma unroll
      for (int t = 0; t < 32; ++t) v[t] = apply_act(v[t], ACT_GELU);
      break;
    case ACT_GELU_TANH:
#pragma unroll
      for (int t = 0; t < 32; ++t) v[t] = apply_act(v[t], ACT_GELU_TANH);
      break;
    case ACT_QUICK_GELU:
#pragma unroll
      for (int t = 0; t < 32; ++t) v[t] = apply_act(v[t], ACT_QUICK_GELU);
      break;
    case ACT_SILU:
#pragma unroll
      for (int t = 0; t < 32; ++t) v[t] = apply_act(v[t], ACT_SILU);
      break;
    default: break;
  }
}

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFF = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;  // + barriers + alignment slack
};

template <int BN, int STAGES, bool TRANS_OUT, bool SWIGLU = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const GemmParams p) {
  using L = SmemLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* s_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);  // [0] abort, [1] is_last

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128
                                 : (2 * BN <= 256) ? 256 : 512;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 128);
    }
    s_flag[0] = 0;
    s_flag[1] = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_kb = (p.K + BK - 1) / BK;

  auto decode_work = [&](int w, int& m_blk, int& n_blk, int& kb0, int& kb1, int& tile, int& split) {
    split = w % p.splits;
    tile = w / p.splits;
    const int per_group = p.group_m * p.num_n;
    const int g = tile / per_group;
    const int first_m = g * p.group_m;
    const int gm = min(p.num_m - first_m, p.group_m);
    const int local = tile - g * per_group;
    m_blk = first_m + local % gm;
    n_blk = local / gm;
    kb0 = split * p.kb_per_split;
    kb1 = min(num_kb, kb0 + p.kb_per_split);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x) {
        int m_blk, n_blk, kb0, kb1, tile, split;
        decode_work(w, m_blk, n_blk, kb0, kb1, tile, split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (s_flag[0] || !mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_EMPTY)) {
            s_flag[0] = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          tma_load_2d(sa, &tma_a, &full_bar[stage], kb * BK, m_blk * BM);
          if constexpr (SWIGLU) {
            // B tile = 128 rows of the gate half + the matching 128 rows of the up half
            tma_load_2d(sb, &tma_b, &full_bar[stage], kb * BK, n_blk * (BN / 2));
            tma_load_2d(sb + L::B_BYTES / 2, &tma_b, &full_bar[stage], kb * BK, p.up_row0 + n_blk * (BN / 2));
          } else {
            tma_load_2d(sb, &tma_b, &full_bar[stage], kb * BK, n_blk * BN);
          }
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // unwind: let every copy that was issued land before the CTA may exit
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
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x) {
        int m_blk, n_blk, kb0, kb1, tile, split;
        decode_work(w, m_blk, n_blk, kb0, kb1, tile, split);
        if (s_flag[0] || !mbar_wait(&acc_empty[acc], acc_phase ^ 1, p.status, ST_TIMEOUT_ACC_EMPTY)) {
          s_flag[0] = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (s_flag[0] || !mbar_wait(&full_bar[stage], phase, p.status, ST_TIMEOUT_FULL)) {
            s_flag[0] = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint64_t da = make_sdesc_sw128(sa);
          const uint64_t db = make_sdesc_sw128(sa + L::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // +32 bytes per K = 16 step inside the 128-byte swizzle row (address field is >> 4)
            tc_mma_f16(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit(&acc_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int lane_group = warp & 3;                 // TMEM lanes this warp may read
    const int row = lane_group * 32 + lane;          // row of the 128 x BN tile
    const int ep_tid = (warp - 2) * 32 + lane;       // 0..127
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int w = blockIdx.x; w < p.total_work; w += gridDim.x) {
      int m_blk, n_blk, kb0, kb1, tile, split;
      decode_work(w, m_blk, n_blk, kb0, kb1, tile, split);
      if (s_flag[0] || !mbar_wait(&acc_full[acc], acc_phase, p.status, ST_TIMEOUT_ACC_FULL)) {
        s_flag[0] = 1;
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (uint32_t(lane_group * 32) << 16) + uint32_t(acc * BN);
      const int gi = m_blk * BM + row;
      const int j0 = n_blk * BN;

      auto finish_chunk = [&](float (&v)[32], int c) {
        // v: 32 consecutive columns of row `gi`, starting at column j0 + 32 c
        const int jb = j0 + c * 32;
        if (gi >= p.M) return;
        float bi = (p.bias != nullptr && p.bias_on_i) ? __bfloat162float(p.bias[gi]) : 0.f;
        if constexpr (!TRANS_OUT) {
          __nv_bfloat16* dst = p.C + (long long)gi * p.ldc_i + jb;
          const bool vec_ok = (jb + 32 <= p.N) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
          if (vec_ok) {
            if (p.bias != nullptr) {
              if (p.bias_on_i) {
#pragma unroll
                for (int t = 0; t < 32; ++t) v[t] += bi;
              } else if ((reinterpret_cast<uintptr_t>(p.bias + jb) & 15) == 0) {
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
            apply_act_chunk(v, p.act);
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
                float a = v[t] + bi;
                if (p.bias != nullptr && !p.bias_on_i) a += __bfloat162float(p.bias[jb + t]);
                dst[t] = __float2bfloat16(apply_act(a, p.act));
              }
            }
          }
        } else {
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            if (jb + t < p.N) {
              float a = v[t] + bi;
              if (p.bias != nullptr && !p.bias_on_i) a += __bfloat162float(p.bias[jb + t]);
              p.C[(long long)gi * p.ldc_i + (long long)(jb + t) * p.ldc_j] = __float2bfloat16(apply_act(a, p.act));
            }
          }
        }
      };

      if constexpr (SWIGLU) {
        // accumulator columns [0, BN/2) = gate, [BN/2, BN) = up; out[:, n_blk * BN/2 + j] = silu(gate_j) * up_j
        const int jo = n_blk * (BN / 2);
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(t_addr + uint32_t(c * 32), rg);
          tmem_ld_32x32(t_addr + uint32_t(BN / 2 + c * 32), ru);
          tmem_ld_wait();
          if (c == BN / 64 - 1) {
            tc_fence_before();
            mbar_arrive(&acc_empty[acc]);
          }
          if (gi < p.M) {
            __nv_bfloat16* dst = p.C + (long long)gi * p.ldc_i + jo + c * 32;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t u[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int t = q * 8 + e * 2;
                const float g0 = __uint_as_float(rg[t]), g1 = __uint_as_float(rg[t + 1]);
                const float a = g0 / (1.f + __expf(-g0)) * __uint_as_float(ru[t]);
                const float b = g1 / (1.f + __expf(-g1)) * __uint_as_float(ru[t + 1]);
                u[e] = pack_bf16(a, b);
              }
              *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(u[0], u[1], u[2], u[3]);
            }
          }
        }
      } else if (p.splits == 1) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_addr + uint32_t(c * 32), r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int t = 0; t < 32; ++t) v[t] = __uint_as_float(r[t]);
          if (c == BN / 32 - 1) {
            // accumulator fully read: hand it back before the global stores
            tc_fence_before();
            mbar_arrive(&acc_empty[acc]);
          }
          finish_chunk(v, c);
        }
      } else {
        // split-K: park the fp32 partial, the last split to arrive reduces
        float* part = p.scratch + ((long long)tile * p.splits + split) * (BM * BN);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_addr + uint32_t(c * 32), r);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 32; ++t) part[(c * 32 + t) * BM + row] = __uint_as_float(r[t]);
        }
        tc_fence_before();
        mbar_arrive(&acc_empty[acc]);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ep_tid == 0) {
          const int old = atomicAdd(&p.counters[tile], 1);
          s_flag[1] = (old == p.splits - 1) ? 1 : 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (s_flag[1]) {
          __threadfence();
          const float* base = p.scratch + (long long)tile * p.splits * (BM * BN);
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            float v[32];
#pragma unroll
            for (int t = 0; t < 32; ++t) v[t] = 0.f;
            for (int s = 0; s < p.splits; ++s) {
              const float* ps = base + (long long)s * (BM * BN);
#pragma unroll
              for (int t = 0; t < 32; ++t) v[t] += __ldcg(&ps[(c * 32 + t) * BM + row]);
            }
            finish_chunk(v, c);
          }
          if (ep_tid == 0) p.counters[tile] = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// =============================================================== host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &ptr, 12000, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || ptr == nullptr)
      throw std::runtime_error("cuTensorMapEncodeTiled is not available from the driver");
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// 2-D bf16 row-major matrix [rows, cols] with row pitch `ld` elements; box = [box_rows, 64 cols], 128B swizzle.
CUtensorMap make_tmap_bf16_2d(const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                              uint32_t box_cols) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) throw std::runtime_error("TMA base must be 16-byte aligned");
  if ((ld * 2) % 16 != 0) throw std::runtime_error("TMA row pitch must be a multiple of 16 bytes");
  CUtensorMap m;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = get_encode()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
  return m;
}

template <int BN, int STAGES, bool TRANS, bool SWIGLU = false>
static void launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                       cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = gemm_bf16_kernel<BN, STAGES, TRANS, SWIGLU>;
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
  kern<<<grid, GEMM_THREADS, L::TOTAL, stream>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("gemm launch: ") + cudaGetErrorString(e));
}

static int g_num_sms = 0;

int gemm_num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_num_sms;
}

size_t gemm_scratch_bytes() { return size_t(GEMM_SCRATCH_TILES) * BM * 256 * sizeof(float); }
size_t gemm_counter_bytes() { return size_t(GEMM_MAX_TILES_SPLIT) * sizeof(int); }

// C[M, N] (ldc) = act(X[M, K] @ W[N, K]^T + bias[N]).  Chooses between the plain
// form (tokens on the 128-row operand) and the swapped, optionally split-K form
// for small M.
void gemm_bf16(const void* x, const void* w, void* c, const void* bias, int M, int N, int K, long long ldx,
               long long ldw, long long ldc, int act, const GemmWorkspace& ws, int sm_limit, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return;
  const int sms = sm_limit > 0 ? sm_limit : gemm_num_sms();
  GemmParams p{};
  p.K = K;
  p.C = reinterpret_cast<__nv_bfloat16*>(c);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.act = act;
  p.status = ws.status;
  p.scratch = ws.scratch;
  p.counters = ws.counters;
  const int num_kb = (K + BK - 1) / BK;
  const bool swapped = (M <= 256);
  if (!swapped && gemm_pairs_mode() &&
      gemm_bf16_2cta(x, w, c, bias, M, N, K, ldx, ldw, ldc, act, sm_limit, ws.status, stream))
    return;
  if (!swapped) {
    // tokens are the 128-row operand
    p.M = M;
    p.N = N;
    p.ldc_i = ldc;
    p.ldc_j = 1;
    p.bias_on_i = 0;
    p.splits = 1;
    p.kb_per_split = num_kb;
    p.num_m = (M + BM - 1) / BM;
    p.group_m = 16;
    CUtensorMap ta = make_tmap_bf16_2d(x, M, K, ldx, BM, BK);
    if (act == ACT_SWIGLU) {
      // w = [gate; up] stacked ([N, K], N = 2 x width); c is [M, N / 2]
      constexpr int BN = 256;
      const int width = N / 2;
      if (N % 256 != 0 || ldc % 8 != 0 || (reinterpret_cast<uintptr_t>(c) & 15) != 0 || bias != nullptr)
        throw std::runtime_error("fused SwiGLU GEMM needs N % 256 == 0, a 16-byte aligned output and no bias");
      p.N = width;
      p.act = ACT_NONE;
      p.up_row0 = width;
      p.num_n = width / (BN / 2);
      p.total_work = p.num_m * p.num_n;
      CUtensorMap tb = make_tmap_bf16_2d(w, N, K, ldw, BN / 2, BK);
      launch_one<BN, 4, false, true>(ta, tb, p, std::min(p.total_work, sms), stream);
      return;
    }
    if (N >= 256 || N % 256 == 0) {
      constexpr int BN = 256;
      p.num_n = (N + BN - 1) / BN;
      p.total_work = p.num_m * p.num_n;
      CUtensorMap tb = make_tmap_bf16_2d(w, N, K, ldw, BN, BK);
      launch_one<BN, 4, false>(ta, tb, p, std::min(p.total_work, sms), stream);
    } else {
      constexpr int BN = 128;
      p.num_n = (N + BN - 1) / BN;
      p.total_work = p.num_m * p.num_n;
      CUtensorMap tb = make_tmap_bf16_2d(w, N, K, ldw, BN, BK);
      launch_one<BN, 6, false>(ta, tb, p, std::min(p.total_work, sms), stream);
    }
    return;
  }
  if (act == ACT_SWIGLU) throw std::runtime_error("fused SwiGLU GEMM is for M > 256; use linear_silu_mul below that");
  // decode-size batch with more 256-row tiles than SMs (the LM head): equal spans of (tile, K block) units per SM
  if (M <= 128 && streamk_enabled() && (N + 255) / 256 >= sms &&
      gemm_streamk_bf16(x, w, c, bias, M, N, K, ldx, ldw, ldc, act, false, ws, sm_limit, stream))
    return;
  // decode-size batch: weight-streaming kernel (gemm_skinny.cu)
  gemm_skinny_bf16(x, w, c, bias, M, N, K, ldx, ldw, ldc, act, ws, sm_limit, 0, true, stream);
}

}  // namespace fc
