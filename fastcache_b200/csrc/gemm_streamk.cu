// Persistent weight-streaming GEMM for decode-size batches (M <= 128 tokens) whose result is finished in the
// kernel: y = act(x W^T + bias), or y = silu(x Wg^T) * (x Wu^T) for a stacked [gate; up] weight.
//
// gemm_skinny.cu deals the (row tile, K split) pairs out as CTAs.  When there are more row tiles than SMs (the LM
// head: 594 tiles of 256 rows on 148 SMs) the last wave is nearly empty, and when there are fewer (gate/up: 96)
// the K splits leave fp32 partial sums [splits, M, N] for a second kernel.  Here the work is one list of
// (row tile, 64-wide K block) units, cut into `grid` equal contiguous spans, one per CTA, one CTA per SM
// ("stream-K"), so every SM streams the same number of weight bytes:
//
//   warp 0     TMA producer: walks the span's units, W tile 256 x 64 and x tile BN x 64 per stage (the ring of
//              stages runs on across row tiles); the first weight tiles are requested before the previous
//              kernel of the stream has finished (programmatic dependent launch)
//   warp 1     tcgen05.mma issuer; two accumulator buffers in tensor memory (2 x 2 x BN columns), so the
//              epilogue of one row tile runs under the main loop of the next
//   warps 2-5  epilogue: tcgen05.ld, then
//                * the CTA whose span holds the END of the row tile's K range owns the tile: it adds the partial
//                  sums of the CTAs that hold the rest (read from scratch through L2), applies bias / activation
//                  / SwiGLU and writes bf16
//                * any other CTA writes its fp32 partial sums to its scratch slot and bumps the tile's arrival
//                  counter
//
// A span is walked from its LAST unit to its first.  The tile that crosses the end of CTA c's span is therefore the
// first thing CTA c works on, and the same tile is the last thing CTA c + 1 (its owner, or another contributor)
// works on: an owner only ever waits for CTAs with a lower index, which started no later than itself and did
// the awaited work first.  The wait is bounded all the same (status ST_TIMEOUT_GRID).  Each CTA contributes to at
// most one tile it does not own (the one crossing the end of its span), so one scratch slot per CTA is enough.
// The counters are zero before the first launch and the owner leaves them zero.
//
// SwiGLU: a row tile is 128 gate rows and the matching 128 up rows (two 128-row MMAs that share the x tile), so
// gate and up of one output element sit in the same TMEM lane and the epilogue needs nothing else.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <stdexcept>
#include <string>

#include "gemm.h"
#include "launch.h"
#include "ptx.cuh"

namespace fc {

namespace {

constexpr int SP_ROWS = 256;
constexpr int SP_BK = 64;
constexpr int SP_THREADS = 192;

struct StreamKParams {
  int Nw, Mtok, K;
  int num_kb, tiles, total_units, units_per_cta;
  __nv_bfloat16* out;
  long long ldc;
  const __nv_bfloat16* bias;
  int act;
  int swiglu;
  float* partial;       // [grid][2][BN][128] fp32
  int* counters;        // [tiles]
  uint32_t* status;
};

__device__ __forceinline__ float sp_act(float v, int act) {
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

__device__ __forceinline__ void sp_epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ int sp_ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <int BN, int STAGES>
struct SpSmem {
  static constexpr int A_BYTES = SP_ROWS * SP_BK * 2;
  static constexpr int B_BYTES = BN * SP_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFF = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

// part i of a span [u0, u1): row tile and K-block range, from the last tile of the span to the first
struct SpPart {
  int tile, ka, kb;
};
__device__ __forceinline__ SpPart sp_part(int i, int u0, int u1, int num_kb) {
  SpPart r;
  r.tile = (u1 - 1) / num_kb - i;
  r.ka = max(u0, r.tile * num_kb) - r.tile * num_kb;
  r.kb = min(u1, (r.tile + 1) * num_kb) - r.tile * num_kb;
  return r;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(SP_THREADS, 1)
gemm_streamk_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x,
                    const StreamKParams p) {
  using L = SpSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;       // [2]
  uint64_t* acc_empty = acc_full + 2;            // [2], 128 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* s_flag = s_abort + 1;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t BUF_COLS = 2 * BN;                                   // gate / first half, up / second half
  constexpr uint32_t TMEM_COLS = (2 * BUF_COLS <= 128) ? 128 : (2 * BUF_COLS <= 256) ? 256 : 512;
  const int cta = blockIdx.x;
  const int u0 = cta * p.units_per_cta;
  const int u1 = min(p.total_units, u0 + p.units_per_cta);
  const int nparts = u1 > u0 ? (u1 - 1) / p.num_kb - u0 / p.num_kb + 1 : 0;
  const int row_step = p.swiglu ? 128 : SP_ROWS;
  const int row1_off = p.swiglu ? p.Nw / 2 : 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 128);
    }
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
  if (!is_producer) pdl_wait();            // x, the scratch and the output belong to earlier kernels until here

  if (warp == 0) {
    if (lane == 0 && nparts > 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      // the weights never change during serving: the first tiles are requested before the wait on the previous
      // kernel, the matching activation tiles right after it
      const int total = u1 - u0;
      const int npre = min(STAGES, total);
      {
        int n = 0;
        for (int i = 0; i < nparts && n < npre; ++i) {
          const SpPart pt = sp_part(i, u0, u1, p.num_kb);
          for (int kb = pt.ka; kb < pt.kb && n < npre; ++kb, ++n) {
            uint8_t* sa = smem + n * L::STAGE_BYTES;
            mbar_expect_tx(&full_bar[n], L::STAGE_BYTES);
            tma_load_2d(sa, &tma_w, &full_bar[n], kb * SP_BK, pt.tile * row_step);
            tma_load_2d(sa + L::A_BYTES / 2, &tma_w, &full_bar[n], kb * SP_BK, pt.tile * row_step + row1_off);
          }
        }
      }
      pdl_wait();
      asm volatile("fence.proxy.async.global;" ::: "memory");   // x: ordinary stores before, TMA reads now
      int n = 0;
      for (int i = 0; i < nparts && ok; ++i) {
        const SpPart pt = sp_part(i, u0, u1, p.num_kb);
        for (int kb = pt.ka; kb < pt.kb; ++kb, ++n) {
          if (n < npre) {
            tma_load_2d(smem + n * L::STAGE_BYTES + L::A_BYTES, &tma_x, &full_bar[n], kb * SP_BK, 0);
            if (n + 1 == npre) {
              stage = npre == STAGES ? 0 : npre;
              phase = npre == STAGES ? 1u : 0u;
            }
            issued = n + 1;
            continue;
          }
          if (*s_abort || !mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_EMPTY)) {
            *s_abort = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          tma_load_2d(sa, &tma_w, &full_bar[stage], kb * SP_BK, pt.tile * row_step);
          tma_load_2d(sa + L::A_BYTES / 2, &tma_w, &full_bar[stage], kb * SP_BK, pt.tile * row_step + row1_off);
          tma_load_2d(sa + L::A_BYTES, &tma_x, &full_bar[stage], kb * SP_BK, 0);
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // wait for the copies in flight before the CTA may exit
        int s = stage;
        uint32_t ph = phase;
        for (int k = 0; k < min(issued, STAGES); ++k) {
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
      for (int i = 0; i < nparts && ok; ++i) {
        const SpPart pt = sp_part(i, u0, u1, p.num_kb);
        const int buf = i & 1;
        if (*s_abort || !mbar_wait(&acc_empty[buf], ((uint32_t(i) >> 1) & 1u) ^ 1u, p.status, ST_TIMEOUT_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t acc = tmem_base + uint32_t(buf) * BUF_COLS;
        for (int kb = pt.ka; kb < pt.kb; ++kb) {
          if (*s_abort || !mbar_wait(&full_bar[stage], phase, p.status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint64_t da0 = make_sdesc_sw128(sa);
          const uint64_t da1 = make_sdesc_sw128(sa + L::A_BYTES / 2);
          const uint64_t db = make_sdesc_sw128(sa + L::A_BYTES);
#pragma unroll
          for (int k = 0; k < SP_BK / 16; ++k) {
            const uint32_t accum = (kb > pt.ka || k > 0) ? 1u : 0u;
            tc_mma_f16(acc, da0 + uint64_t(2 * k), db + uint64_t(2 * k), idesc, accum);
            tc_mma_f16(acc + BN, da1 + uint64_t(2 * k), db + uint64_t(2 * k), idesc, accum);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit(&acc_full[buf]);
      }
      if (!ok) *s_abort = 1;
    }
  } else {
    // ------------------------------------------------------------------ epilogue (128 threads)
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;
    const int etid = (warp - 2) * 32 + lane;
    const uint32_t t_lane = uint32_t(lane_group * 32) << 16;
    constexpr int SLOT_FLOATS = 2 * BN * 128;
    bool ok = true;
    // every thread walks every part and meets every named barrier, also after a wait that ran out (it then
    // only skips the memory traffic): the 128 threads must not lose step with each other
    for (int i = 0; i < nparts; ++i) {
      const SpPart pt = sp_part(i, u0, u1, p.num_kb);
      const int buf = i & 1;
      if (ok && (*s_abort || !mbar_wait(&acc_full[buf], (uint32_t(i) >> 1) & 1u, p.status, ST_TIMEOUT_ACC_FULL))) {
        ok = false;
        *s_abort = 1;
      }
      tc_fence_after();
      const uint32_t acc = tmem_base + t_lane + uint32_t(buf) * BUF_COLS;
      const bool owner = pt.kb == p.num_kb;
      if (!owner) {
        float* slot = p.partial + (long long)cta * SLOT_FLOATS;
        if (ok) {
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
              uint32_t r[32];
              tmem_ld_32x32(acc + uint32_t(h * BN + c * 32), r);
              tmem_ld_wait();
#pragma unroll
              for (int t = 0; t < 32; ++t)
                if (c * 32 + t < p.Mtok) slot[(h * BN + c * 32 + t) * 128 + row] = __uint_as_float(r[t]);
            }
          }
        }
        tc_fence_before();
        mbar_arrive(&acc_empty[buf]);
        __threadfence();
        sp_epi_bar();
        if (etid == 0 && ok) atomicAdd(p.counters + pt.tile, 1);
      } else {
        // CTAs a .. cta - 1 hold the rest of this tile's K range
        const int a = (pt.tile * p.num_kb) / p.units_per_cta;
        const int need = cta - a;
        if (need > 0) {
          if (etid == 0) {
            bool arrived = false;
            if (ok) {
              const uint64_t limit = status_wait_limit_ns(p.status, 2000000000ull);
              const uint64_t t0 = global_timer_ns();
              uint32_t spins = 0;
              while (true) {
                if (sp_ld_acquire(p.counters + pt.tile) >= need) {
                  arrived = true;
                  break;
                }
                if ((++spins & 63u) == 0u && global_timer_ns() - t0 > limit) break;
              }
              if (!arrived) report(p.status, ST_TIMEOUT_GRID);
              else p.counters[pt.tile] = 0;          // ready for the next launch
            }
            *s_flag = arrived ? 1 : 0;
            __threadfence();
          }
          sp_epi_bar();
          if (*s_flag == 0) ok = false;
          sp_epi_bar();                              // s_flag may be rewritten for the next part after this
        }
        if (ok) {
          const int n0 = pt.tile * row_step + row;               // first-half output feature of this thread
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(acc + uint32_t(c * 32), r0);
            tmem_ld_32x32(acc + uint32_t(BN + c * 32), r1);
            tmem_ld_wait();
            for (int q = a; q < cta; ++q) {
              const float* slot = p.partial + (long long)q * SLOT_FLOATS;
#pragma unroll
              for (int t = 0; t < 32; ++t) {
                if (c * 32 + t < p.Mtok) {
                  r0[t] = __float_as_uint(__uint_as_float(r0[t]) + __ldcg(slot + (c * 32 + t) * 128 + row));
                  r1[t] = __float_as_uint(__uint_as_float(r1[t]) + __ldcg(slot + (BN + c * 32 + t) * 128 + row));
                }
              }
            }
            if (p.swiglu) {
              if (n0 < p.Nw / 2) {
#pragma unroll
                for (int t = 0; t < 32; ++t) {
                  const int tok = c * 32 + t;
                  if (tok < p.Mtok) {
                    const float g = __uint_as_float(r0[t]), u = __uint_as_float(r1[t]);
                    p.out[(long long)tok * p.ldc + n0] = __float2bfloat16(g / (1.f + __expf(-g)) * u);
                  }
                }
              }
            } else {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int n = n0 + h * 128;
                if (n < p.Nw) {
                  const float bi = p.bias != nullptr ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll
                  for (int t = 0; t < 32; ++t) {
                    const int tok = c * 32 + t;
                    if (tok < p.Mtok)
                      p.out[(long long)tok * p.ldc + n] =
                          __float2bfloat16(sp_act(__uint_as_float(h == 0 ? r0[t] : r1[t]) + bi, p.act));
                  }
                }
              }
            }
          }
        }
        tc_fence_before();
        mbar_arrive(&acc_empty[buf]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

int g_streamk = -1;

template <int BN, int STAGES>
void sp_launch(const CUtensorMap& tw, const CUtensorMap& tx, const StreamKParams& p, int grid, cudaStream_t stream) {
  using L = SpSmem<BN, STAGES>;
  auto kern = gemm_streamk_kernel<BN, STAGES>;
  static std::atomic<uint64_t> configured{0};
  int dev = 0;
  cudaGetDevice(&dev);
  const uint64_t bit = 1ull << (dev & 63);
  if (!(configured.load(std::memory_order_relaxed) & bit)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) throw std::runtime_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    configured.fetch_or(bit, std::memory_order_relaxed);
  }
  cudaError_t e = launch_pdl(PDL_SKINNY_GEMM, kern, dim3(grid), dim3(SP_THREADS), size_t(L::TOTAL), stream, tw, tx, p);
  if (e != cudaSuccess) throw std::runtime_error(std::string("stream-K gemm launch: ") + cudaGetErrorString(e));
}

}  // namespace

int streamk_mode() {
  if (g_streamk < 0) {
    const char* e = std::getenv("FC_STREAMK");
    g_streamk = e == nullptr ? 1 : std::max(0, std::min(2, std::atoi(e)));
  }
  return g_streamk;
}
bool streamk_enabled() { return streamk_mode() > 0; }
void set_streamk(int mode) { g_streamk = std::max(0, std::min(2, mode)); }

bool gemm_streamk_bf16(const void* x, const void* w, void* c, const void* bias, int M, int N, int K, long long ldx,
                       long long ldw, long long ldc, int act, bool swiglu, const GemmWorkspace& ws, int sm_limit,
                       cudaStream_t stream) {
  if (M <= 0 || M > 128 || N <= 0 || K <= 0 || ws.scratch == nullptr || ws.counters == nullptr) return false;
  if (swiglu && (N % 256 != 0 || bias != nullptr)) return false;
  const int sms = sm_limit > 0 ? sm_limit : gemm_num_sms();
  const int tiles = swiglu ? N / 256 : (N + SP_ROWS - 1) / SP_ROWS;
  if (tiles > GEMM_MAX_TILES_SPLIT) return false;
  // A tile's partial sums are added by ONE CTA (its owner).  With few row tiles every tile is cut into many spans
  // and that serial reduction costs more than the second kernel it saves: mode 1 leaves such shapes to the split-K
  // + consumer form (at most about three spans per tile here), mode 2 takes everything.
  if (streamk_mode() < 2 && tiles * 3 < sms) return false;
  const int num_kb = (K + SP_BK - 1) / SP_BK;
  const int total = tiles * num_kb;
  const int BN = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  // at least 4 K blocks per CTA; spans of equal length, then only as many CTAs as have a span
  int grid = std::max(1, std::min(sms, total / 4));
  const int upc = (total + grid - 1) / grid;
  grid = (total + upc - 1) / upc;
  if ((size_t)grid * 2 * BN * 128 * sizeof(float) > gemm_scratch_bytes()) return false;
  StreamKParams p{};
  p.Nw = N;
  p.Mtok = M;
  p.K = K;
  p.num_kb = num_kb;
  p.tiles = tiles;
  p.total_units = total;
  p.units_per_cta = upc;
  p.out = reinterpret_cast<__nv_bfloat16*>(c);
  p.ldc = ldc;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.act = act;
  p.swiglu = swiglu ? 1 : 0;
  p.partial = ws.scratch;
  p.counters = ws.counters;
  p.status = ws.status;
  const CUtensorMap tw = make_tmap_bf16_2d(w, N, K, ldw, 128, SP_BK);
  const CUtensorMap tx = make_tmap_bf16_2d(x, M, K, ldx, BN, SP_BK);
  if (BN == 32) sp_launch<32, 6>(tw, tx, p, grid, stream);
  else if (BN == 64) sp_launch<64, 5>(tw, tx, p, grid, stream);
  else sp_launch<128, 4>(tw, tx, p, grid, stream);
  return true;
}

}  // namespace fc
