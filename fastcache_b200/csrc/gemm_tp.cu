// Tensor-parallel GEMMs fused with their collective (prefill sizes), over symmetric memory.
//
// Token rows are split into `tp` contiguous chunks of `chunk_rows` (a multiple of 128); rank r owns
// chunk r: it holds the residual stream of those rows and is the one that normalises them.
//
// MODE_RS  (row-parallel projection: o_proj, down_proj)
//   y_partial[T, H] = x[T, K/tp] @ W[H, K/tp]^T on every rank.  The tcgen05 main loop is the one of
//   gemm.cu (TMA -> smem ring -> tcgen05.mma -> TMEM); the epilogue stores each 128-row tile of the
//   partial sums straight into the OWNER's staging buffer (slot = source rank) with peer stores, remote
//   owners first so the NVLink traffic overlaps the rest of the GEMM.  When a rank has written all
//   tiles of an owner it raises that owner's flag (release, system scope).  After its own tiles every
//   CTA turns to the rows this rank owns: it waits (bounded) for the flags of all source ranks, sums
//   the tp partials, adds the residual (updated in place), applies RMSNorm and stores the normalised
//   rows into the gathered activation buffer of EVERY rank; the last CTA raises the "gathered" flag on
//   every rank.  That is reduce-scatter + residual add + RMSNorm + the send half of the all-gather in
//   the GEMM kernel.
//
// MODE_AG  (column-parallel projection that follows: qkv_proj, gate_up_proj)
//   A is the gathered activation buffer in local memory.  The TMA producer waits (bounded) for the
//   "gathered" flag of a chunk's owner before it loads the first tile of that chunk and starts with
//   its own chunk, so the GEMM runs while later chunks are still arriving.
//
// MODE_RS, pipelined form (FC_TP_PIPELINE=1; off by default, it measured no faster than the one reduction phase
// after the GEMM): the tiles are walked row group by row group across the owners (group g of
// owner rank + 1, of rank + 2, ..., of this rank, then group g + 1, ...), every rank counts the tiles it has
// delivered per (owner, 128-row group) and raises a flag per group, and six extra warps per CTA ("reducers")
// wait for the flags of the groups this rank owns and reduce + normalise + send them while the main loop is still
// working on later groups.  Only the last groups' reduction is left after the GEMM instead of the whole chunk's.
//
// With NVSwitch multicast addresses for the staging and gathered buffers (NVLS; FC_TP_NVLS=0 turns it off) the
// pipelined form moves fewer bytes: the epilogue writes its partial tiles into this rank's OWN staging buffer
// ([M][N], plain local stores), the owner of a row sums the `tp` copies inside the switch (multimem.ld_reduce:
// one row crosses the owner's link once instead of tp - 1 times) and publishes the normalised row with one
// multimem.st (one row leaves the owner once instead of tp - 1 times).
//
// No TMA touches peer memory and no load is multicast; remote data always lands in the consumer's own
// memory through ordinary stores first.  Every wait is bounded and reports through the status word.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <stdexcept>
#include <string>

#include "comm.h"
#include "gemm.h"
#include "ptx.cuh"

namespace fc {

constexpr int TP_BM = 128;
constexpr int TP_BK = 64;
constexpr int TP_BN = 256;
constexpr int TP_STAGES = 4;
constexpr int TP_THREADS = 192;
constexpr int MODE_RS = 1;
constexpr int MODE_AG = 2;
constexpr int MODE_AG_SWIGLU = 3;   // MODE_AG on w = [gate; up] with silu(gate) * up applied in the epilogue

struct TpGemmParams {
  int M, N, K;                 // tokens, output features, reduction length (local)
  int num_m, num_n, group_m;
  int total_tiles;
  int tp, rank, chunk_rows, blocks_per_chunk, rot;
  uint32_t epoch;
  uint32_t* status;
  int up_row0;                 // MODE_AG_SWIGLU: first row of the up half of w (= output width)
  // MODE_AG: plain output
  __nv_bfloat16* C;
  long long ldc;
  const uint32_t* gathered_flags;             // local [tp]: raised by each owner when its rows have landed
  // MODE_RS
  __nv_bfloat16* stage_peer[COMM_MAX_WORLD];  // staging buffer of every rank: [tp][chunk_rows][N]
  uint32_t* rs_flag_peer[COMM_MAX_WORLD];     // [tp] words on every rank: "source s has delivered"
  const __nv_bfloat16* stage_local;           // this rank's staging buffer
  const uint32_t* rs_flags_local;
  int* owner_done;                            // local [tp + 1] counters (last = CTAs done with phase 2)
  __nv_bfloat16* residual;                    // [rows owned, N], updated in place
  const __nv_bfloat16* norm_w;
  float eps;
  __nv_bfloat16* xg_peer[COMM_MAX_WORLD];     // gathered activation buffer of every rank: [>= M, N]
  uint32_t* gathered_flag_peer[COMM_MAX_WORLD];
  // MODE_RS, pipelined form (see the header): per 128-row group instead of per chunk
  int pipelined;
  int max_groups;                             // row groups per chunk that the flag / counter arrays hold
  int* group_done;                            // local [tp][max_groups]: tiles of (owner, group) delivered by this rank
  uint32_t* group_flag_peer[COMM_MAX_WORLD];  // [max_groups][COMM_MAX_WORLD] words on every rank: "source s delivered group g"
  const uint32_t* group_flags_local;
  // NVLS form of the pipelined kernel: the partial sums stay in this rank's own staging buffer, laid out [M][N];
  // the owner of a row sums all ranks' copies with multimem.ld_reduce through the multicast address of the
  // staging buffers and publishes the normalised row with one multimem.st to every rank's gathered buffer
  const __nv_bfloat16* stage_mc;              // nullptr: peer stores and local sums
  __nv_bfloat16* xg_mc;
  __nv_bfloat16* stage_rw;                    // this rank's staging buffer, writable
};

__device__ __forceinline__ void tp_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t tp_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// bounded wait for a flag to reach `epoch` (epochs only grow)
__device__ __forceinline__ bool tp_wait_flag(const uint32_t* flag, uint32_t epoch, uint32_t* status) {
  const uint64_t t0 = global_timer_ns();
  uint64_t limit = FC_PEER_WAIT_LIMIT_NS;
  for (uint32_t i = 0; i < (1u << 28); ++i) {
    if (int32_t(tp_ld_acquire(flag) - epoch) >= 0) return true;
    __nanosleep(40);
    if ((i & 255u) == 255u) {
      if (i == 255u) limit = peer_wait_limit_ns(status);
      if (global_timer_ns() - t0 > limit) break;
    }
  }
  report(status, ST_TIMEOUT_PEER);
  return false;
}

__device__ __forceinline__ uint4 tp_multimem_ld_reduce(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void tp_multimem_st(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// The NVLS form of the row reduction below: one multimem.ld_reduce per 16 bytes instead of `tp` loads, one
// multimem.st instead of `tp` stores.  U pieces per lane in flight.
template <int U>
__device__ __forceinline__ void tp_reduce_rows_nvls(const TpGemmParams& p, int row0, int r_begin, int r_end, int r_step,
                                                    int lane) {
  const int chunks = p.N >> 3;
  for (int r = r_begin; r < r_end; r += r_step) {
    __nv_bfloat16* res_row = p.residual + (long long)r * p.N;
    const long long off_row = (long long)(row0 + r) * p.N;
    float ss = 0.f;
    for (int i0 = lane; i0 < chunks; i0 += 32 * U) {
      uint4 sum[U], ru[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = i0 + 32 * u;
        if (idx < chunks) {
          sum[u] = tp_multimem_ld_reduce(p.stage_mc + off_row + idx * 8);
          ru[u] = *reinterpret_cast<const uint4*>(res_row + idx * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = i0 + 32 * u;
        if (idx < chunks) {
          const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&sum[u]);
          const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&ru[u]);
          uint4 su;
          uint32_t* sw = reinterpret_cast<uint32_t*>(&su);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 a = __bfloat1622float2(ah[i]), f = __bfloat1622float2(rh[i]);
            sw[i] = pack_bf16(a.x + f.x, a.y + f.y);
          }
          *reinterpret_cast<uint4*>(res_row + idx * 8) = su;
          const __nv_bfloat162* sh = reinterpret_cast<const __nv_bfloat162*>(&su);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(sh[i]);
            ss += f.x * f.x + f.y * f.y;
          }
        }
      }
    }
    const float inv = rsqrtf(warp_sum(ss) / float(p.N) + p.eps);
    for (int i0 = lane; i0 < chunks; i0 += 32 * U) {
      uint4 su[U], gu[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = i0 + 32 * u;
        if (idx < chunks) {
          su[u] = *reinterpret_cast<const uint4*>(res_row + idx * 8);
          gu[u] = *reinterpret_cast<const uint4*>(p.norm_w + idx * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = i0 + 32 * u;
        if (idx < chunks) {
          const __nv_bfloat162* sh = reinterpret_cast<const __nv_bfloat162*>(&su[u]);
          const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gu[u]);
          uint4 ou;
          uint32_t* ow = reinterpret_cast<uint32_t*>(&ou);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(sh[i]);
            const float2 g2 = __bfloat1622float2(gh[i]);
            const float a = __bfloat162float(__float2bfloat16(f.x * inv)) * g2.x;
            const float b = __bfloat162float(__float2bfloat16(f.y * inv)) * g2.y;
            ow[i] = pack_bf16(a, b);
          }
          tp_multimem_st(p.xg_mc + off_row + idx * 8, ou);
        }
      }
    }
  }
}

// Phase 2 of MODE_RS for the rows this rank owns.  One warp per row, U 16-byte pieces per lane in
// flight: pass 1 sums the tp partial rows and the residual (written back), pass 2 re-reads the new
// residual (the lane's own lines), scales it and stores the row into every rank's gathered buffer as
// full 512-byte warp stores.
template <int TPMAX, int U>
__device__ __forceinline__ void tp_reduce_rows(const TpGemmParams& p, int row0, int r_begin, int r_end, int r_step,
                                               int lane) {
  const int chunks = p.N >> 3;                         // 16-byte pieces per row
  for (int r = r_begin; r < r_end; r += r_step) {
    __nv_bfloat16* res_row = p.residual + (long long)r * p.N;
    float ss = 0.f;
    for (int i0 = lane; i0 < chunks; i0 += 32 * U) {
      uint4 part[U][TPMAX];
      uint4 ru[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = i0 + 32 * u;
        if (idx < chunks) {
#pragma unroll
          for (int s = 0; s < TPMAX; ++s)
            if (s < p.tp)
              part[u][s] = __ldcg(reinterpret_cast<const uint4*>(
                  p.stage_local + ((long long)s * p.chunk_rows + r) * p.N + idx * 8));
          ru[u] = *reinterpret_cast<const uint4*>(res_row + idx * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = i0 + 32 * u;
        if (idx < chunks) {
          float acc8[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) acc8[i] = 0.f;
#pragma unroll
          for (int s = 0; s < TPMAX; ++s) {
            if (s < p.tp) {
              const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&part[u][s]);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(h2[i]);
                acc8[2 * i] += f.x;
                acc8[2 * i + 1] += f.y;
              }
            }
          }
          const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&ru[u]);
          uint4 su;
          uint32_t* sw = reinterpret_cast<uint32_t*>(&su);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(rh[i]);
            sw[i] = pack_bf16(acc8[2 * i] + f.x, acc8[2 * i + 1] + f.y);
          }
          *reinterpret_cast<uint4*>(res_row + idx * 8) = su;
          const __nv_bfloat162* sh = reinterpret_cast<const __nv_bfloat162*>(&su);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(sh[i]);
            ss += f.x * f.x + f.y * f.y;
          }
        }
      }
    }
    const float inv = rsqrtf(warp_sum(ss) / float(p.N) + p.eps);
    const long long off_row = (long long)(row0 + r) * p.N;
    for (int i0 = lane; i0 < chunks; i0 += 32 * U) {
      uint4 su[U], gu[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = i0 + 32 * u;
        if (idx < chunks) {
          su[u] = *reinterpret_cast<const uint4*>(res_row + idx * 8);
          gu[u] = *reinterpret_cast<const uint4*>(p.norm_w + idx * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = i0 + 32 * u;
        if (idx < chunks) {
          const __nv_bfloat162* sh = reinterpret_cast<const __nv_bfloat162*>(&su[u]);
          const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gu[u]);
          uint4 ou;
          uint32_t* ow = reinterpret_cast<uint32_t*>(&ou);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(sh[i]);
            const float2 g2 = __bfloat1622float2(gh[i]);
            const float a = __bfloat162float(__float2bfloat16(f.x * inv)) * g2.x;
            const float b = __bfloat162float(__float2bfloat16(f.y * inv)) * g2.y;
            ow[i] = pack_bf16(a, b);
          }
#pragma unroll
          for (int d = 0; d < TPMAX; ++d)
            if (d < p.tp) *reinterpret_cast<uint4*>(p.xg_peer[d] + off_row + idx * 8) = ou;
        }
      }
    }
  }
}

constexpr int TP_REDUCERS = 6;                      // reducer warps per CTA (pipelined MODE_RS)
constexpr int TP_THREADS_RS = TP_THREADS + 32 * TP_REDUCERS;

// PIPE (MODE_RS only): the pipelined form with reducer warps; both forms are built so that they can be compared
// NVLS (with PIPE): sums and broadcasts through the NVSwitch multicast addresses
template <int MODE, bool PIPE = false, bool NVLS = false>
__global__ void __launch_bounds__(PIPE ? TP_THREADS_RS : TP_THREADS, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               const TpGemmParams p) {
  constexpr int A_BYTES = TP_BM * TP_BK * 2, B_BYTES = TP_BN * TP_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + TP_STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + TP_STAGES;
  uint64_t* acc_full = empty_bar + TP_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* s_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);   // [0] abort, [1] scratch
  // per epilogue warp: 32 rows x 64 columns of bf16 output on their way from "one row per lane" to
  // "eight lanes per 128-byte row piece" (row pitch 144 bytes keeps both phases free of bank conflicts)
  uint8_t* out_stage = smem + TP_STAGES * STAGE_BYTES + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < TP_STAGES; ++s) {
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
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_kb = (p.K + TP_BK - 1) / TP_BK;

  // tile -> (m_blk, n_blk): grouped raster, then the m-block order is rotated by `rot` blocks so that
  // MODE_RS starts with the chunk of rank + 1 (own chunk last) and MODE_AG with its own chunk
  auto decode_tile = [&](int tile, int& m_blk, int& n_blk) {
    if (PIPE) {
      // row group by row group across the owners, own chunk last within a group
      n_blk = tile % p.num_n;
      const int q = tile / p.num_n;
      const int owner = (p.rank + 1 + q % p.tp) % p.tp;
      m_blk = owner * p.blocks_per_chunk + q / p.tp;
      return;
    }
    const int padded = p.tp * p.blocks_per_chunk;            // >= num_m; blocks >= num_m are skipped
    const int per_group = p.group_m * p.num_n;
    const int g = tile / per_group;
    const int first_m = g * p.group_m;
    const int gm = min(padded - first_m, p.group_m);
    const int local = tile - g * per_group;
    const int m_lin = first_m + local % gm;
    n_blk = local / gm;
    m_blk = (m_lin + p.rot) % padded;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t seen = 0;                                   // owners whose "gathered" flag was observed
      bool ok = true;
      for (int w = blockIdx.x; w < p.total_tiles && ok; w += gridDim.x) {
        int m_blk, n_blk;
        decode_tile(w, m_blk, n_blk);
        if (m_blk >= p.num_m) continue;                    // padding block of the rotated order
        if (MODE != MODE_RS) {
          const int owner = m_blk / p.blocks_per_chunk;
          if (owner != p.rank && !(seen & (1u << owner))) {
            if (!tp_wait_flag(p.gathered_flags + owner, p.epoch, p.status)) {
              s_flag[0] = 1;
              break;
            }
            seen |= 1u << owner;
            asm volatile("fence.proxy.async.global;" ::: "memory");   // peer stores -> TMA reads
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (s_flag[0] || !mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_EMPTY)) {
            s_flag[0] = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          tma_load_2d(sa, &tma_a, &full_bar[stage], kb * TP_BK, m_blk * TP_BM);
          if (MODE == MODE_AG_SWIGLU) {
            // B tile = 128 rows of this rank's gate weights + the matching 128 rows of its up weights
            tma_load_2d(sa + A_BYTES, &tma_b, &full_bar[stage], kb * TP_BK, n_blk * (TP_BN / 2));
            tma_load_2d(sa + A_BYTES + B_BYTES / 2, &tma_b, &full_bar[stage], kb * TP_BK,
                        p.up_row0 + n_blk * (TP_BN / 2));
          } else {
            tma_load_2d(sa + A_BYTES, &tma_b, &full_bar[stage], kb * TP_BK, n_blk * TP_BN);
          }
          if (++stage == TP_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TP_BM, TP_BN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.total_tiles && ok; w += gridDim.x) {
        int m_blk, n_blk;
        decode_tile(w, m_blk, n_blk);
        if (m_blk >= p.num_m) continue;
        if (s_flag[0] || !mbar_wait(&acc_empty[acc], acc_phase ^ 1, p.status, ST_TIMEOUT_ACC_EMPTY)) {
          s_flag[0] = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(acc * TP_BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (s_flag[0] || !mbar_wait(&full_bar[stage], phase, p.status, ST_TIMEOUT_FULL)) {
            s_flag[0] = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint64_t da = make_sdesc_sw128(sa), db = make_sdesc_sw128(sa + A_BYTES);
#pragma unroll
          for (int k = 0; k < TP_BK / 16; ++k)
            tc_mma_f16(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit(&empty_bar[stage]);
          if (++stage == TP_STAGES) {
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
  } else if (warp < 6) {
    const int lane_group = warp & 3;
    const int ep_tid = (warp - 2) * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int w = blockIdx.x; w < p.total_tiles; w += gridDim.x) {
      int m_blk, n_blk;
      decode_tile(w, m_blk, n_blk);
      if (m_blk >= p.num_m) continue;
      if (s_flag[0] || !mbar_wait(&acc_full[acc], acc_phase, p.status, ST_TIMEOUT_ACC_FULL)) {
        s_flag[0] = 1;
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (uint32_t(lane_group * 32) << 16) + uint32_t(acc * TP_BN);
      const int owner = m_blk / p.blocks_per_chunk;
      const int gi0 = m_blk * TP_BM + lane_group * 32;    // first token row of this warp's 32 rows
      // row `gi0 + rr` of the output lives at dst0 + rr * ld
      __nv_bfloat16* dst0;
      long long ld;
      if (MODE == MODE_RS) {
        ld = p.N;
        if (NVLS)
          dst0 = p.stage_rw + (long long)gi0 * p.N;          // NVLS form: this rank's own buffer, [M][N]
        else
          dst0 = p.stage_peer[owner] + ((long long)p.rank * p.chunk_rows + (gi0 - owner * p.chunk_rows)) * p.N;
      } else {
        ld = p.ldc;
        dst0 = p.C + (long long)gi0 * p.ldc;
      }
      uint8_t* stg = out_stage + (warp - 2) * (32 * 144);
      // SwiGLU: accumulator columns [0, 128) = gate, [128, 256) = up, 128 output columns per tile
      constexpr int OUT_COLS = (MODE == MODE_AG_SWIGLU) ? TP_BN / 2 : TP_BN;
#pragma unroll 1
      for (int c2 = 0; c2 < OUT_COLS / 64; ++c2) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld_32x32(t_addr + uint32_t(c2 * 64 + half * 32), r);
          if (MODE == MODE_AG_SWIGLU) {
            uint32_t ru[32];
            tmem_ld_32x32(t_addr + uint32_t(TP_BN / 2 + c2 * 64 + half * 32), ru);
            tmem_ld_wait();
#pragma unroll
            for (int t = 0; t < 32; ++t) {
              const float g = __uint_as_float(r[t]);
              r[t] = __float_as_uint(g / (1.f + __expf(-g)) * __uint_as_float(ru[t]));
            }
          } else {
            tmem_ld_wait();
          }
          if (c2 == OUT_COLS / 64 - 1 && half == 1) {
            tc_fence_before();
            mbar_arrive(&acc_empty[acc]);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_bf16(__uint_as_float(r[q * 8 + 0]), __uint_as_float(r[q * 8 + 1]));
            u.y = pack_bf16(__uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3]));
            u.z = pack_bf16(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5]));
            u.w = pack_bf16(__uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7]));
            *reinterpret_cast<uint4*>(stg + lane * 144 + half * 64 + q * 16) = u;
          }
        }
        __syncwarp();
        // eight lanes write one 128-byte piece of a row: full lines towards HBM or NVLink
        const int jb = n_blk * OUT_COLS + c2 * 64 + (lane & 7) * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = (lane >> 3) + 4 * i;
          const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 144 + (lane & 7) * 16);
          if (gi0 + rr < p.M && jb < p.N) *reinterpret_cast<uint4*>(dst0 + (long long)rr * ld + jb) = v;
        }
        __syncwarp();
      }
      if (MODE == MODE_RS) {
        // this tile is delivered: one thread makes the CTA's stores visible system-wide and counts the
        // tile; the owner's flag goes up after the last one
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ep_tid == 0) {
          __threadfence_system();
          if (PIPE) {
            const int g = m_blk - owner * p.blocks_per_chunk;
            const int old = atomicAdd(&p.group_done[owner * p.max_groups + g], 1);
            if (old + 1 == p.num_n) {
              __threadfence_system();
              tp_st_release(p.group_flag_peer[owner] + (size_t)g * COMM_MAX_WORLD + p.rank, p.epoch);
            }
          } else {
            const int first = owner * p.blocks_per_chunk;
            const int nblk = max(0, min(p.num_m - first, p.blocks_per_chunk));
            const int old = atomicAdd(&p.owner_done[owner], 1);
            if (old + 1 == nblk * p.num_n) {
              __threadfence_system();
              tp_st_release(p.rs_flag_peer[owner] + p.rank, p.epoch);
            }
          }
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  } else if (PIPE) {
    // ------------------------------------------------ reducers (warps 6-11): the rows this rank owns
    // The rows are dealt out one by one over all reducer warps of the grid, so the 128 rows of a group go to 128
    // different warps: what is left when the main loop ends (the last group of every owner completes only then) is
    // one row per warp, not a group per CTA.  A warp takes its rows in rising order and waits for the flags of a
    // row's group when it enters a new group.
    const int rw = warp - 6;
    const int row0r = p.rank * p.chunk_rows;
    const int my_rows_r = max(0, min(p.M - row0r, p.chunk_rows));
    const int stride = int(gridDim.x) * TP_REDUCERS;
    int seen_group = -1;
    for (int r = rw * int(gridDim.x) + int(blockIdx.x); r < my_rows_r; r += stride) {
      const int g = r / TP_BM;
      if (g != seen_group) {
        bool ok = true;
        if (lane < p.tp)
          ok = !s_flag[0] && tp_wait_flag(p.group_flags_local + (size_t)g * COMM_MAX_WORLD + lane, p.epoch, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          s_flag[0] = 1;
          break;
        }
        seen_group = g;
      }
      if (NVLS) {
        tp_reduce_rows_nvls<4>(p, row0r, r, r + 1, 1, lane);
        continue;
      }
      // (fewer pieces in flight than the one-phase form: this kernel has the main loop's state live as well)
      if (p.tp <= 2) tp_reduce_rows<2, 2>(p, row0r, r, r + 1, 1, lane);
      else if (p.tp <= 4) tp_reduce_rows<4, 1>(p, row0r, r, r + 1, 1, lane);
      else tp_reduce_rows<8, 1>(p, row0r, r, r + 1, 1, lane);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (MODE != MODE_RS) return;

  // ------------------------------------------------------------------ phase 2: rows owned by this rank
  const int row0 = p.rank * p.chunk_rows;
  const int my_rows = max(0, min(p.M - row0, p.chunk_rows));
  if (!PIPE && my_rows > 0 && !s_flag[0]) {
    if (threadIdx.x < p.tp) {
      if (!tp_wait_flag(p.rs_flags_local + threadIdx.x, p.epoch, p.status)) s_flag[0] = 1;
    }
    __syncthreads();
    if (!s_flag[0]) {
      constexpr int WARPS = TP_THREADS / 32;             // (the reducer warps of the pipelined form are not here)
      const int rb = blockIdx.x * WARPS + warp, rs = gridDim.x * WARPS;
      if (warp < WARPS) {
        if (p.tp <= 2) tp_reduce_rows<2, 8>(p, row0, rb, my_rows, rs, lane);
        else if (p.tp <= 4) tp_reduce_rows<4, 4>(p, row0, rb, my_rows, rs, lane);
        else tp_reduce_rows<8, 2>(p, row0, rb, my_rows, rs, lane);
      }
    }
  }
  // the last CTA to get here publishes "rows of this rank are gathered" everywhere and resets the counters
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(&p.owner_done[p.tp], 1);
    s_flag[1] = old == int(gridDim.x) - 1 ? 1 : 0;
  }
  __syncthreads();
  if (s_flag[1]) {
    if (PIPE)
      for (int i = threadIdx.x; i < p.tp * p.max_groups; i += blockDim.x) p.group_done[i] = 0;
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int o = 0; o <= p.tp; ++o) p.owner_done[o] = 0;
      __threadfence_system();
      for (int d = 0; d < p.tp; ++d) tp_st_release(p.gathered_flag_peer[d] + p.rank, p.epoch);
    }
  }
}

static int tp_smem_bytes() {
  // operand ring + barriers + output staging (4 epilogue warps x 32 rows x 144 bytes) + alignment slack
  return TP_STAGES * (TP_BM * TP_BK * 2 + TP_BN * TP_BK * 2) + 256 + 4 * 32 * 144 + 1024;
}

static int g_tp_pipeline = -1;
bool tp_pipeline_enabled() {
  if (g_tp_pipeline < 0) {
    const char* e = std::getenv("FC_TP_PIPELINE");
    g_tp_pipeline = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  return g_tp_pipeline == 1;
}
void set_tp_pipeline(bool on) { g_tp_pipeline = on ? 1 : 0; }

static int g_tp_nvls = -1;
bool tp_nvls_enabled() {
  if (g_tp_nvls < 0) {
    const char* e = std::getenv("FC_TP_NVLS");
    g_tp_nvls = (e == nullptr || e[0] != '0') ? 1 : 0;
  }
  return g_tp_nvls == 1;
}
void set_tp_nvls(bool on) { g_tp_nvls = on ? 1 : 0; }

static void fill_common(TpGemmParams& p, int M, int N, int K, int tp, int rank, int chunk_rows, uint32_t epoch,
                        uint32_t* status, bool own_first) {
  p.M = M;
  p.N = N;
  p.K = K;
  p.num_n = (N + TP_BN - 1) / TP_BN;
  p.tp = tp;
  p.rank = rank;
  p.chunk_rows = chunk_rows;
  p.blocks_per_chunk = chunk_rows / TP_BM;
  p.num_m = (M + TP_BM - 1) / TP_BM;
  p.group_m = std::min(16, p.blocks_per_chunk);
  // the rotated order runs over tp * blocks_per_chunk m-blocks; blocks >= num_m are skipped by every role
  p.total_tiles = tp * p.blocks_per_chunk * p.num_n;
  p.rot = ((own_first ? rank : rank + 1) % tp) * p.blocks_per_chunk;
  p.epoch = epoch;
  p.status = status;
}

void gemm_rs_add_norm(const void* x, const void* w, int M, int N, int K, long long ldx, long long ldw,
                      const TpBuffers& b, void* residual, const void* norm_w, float eps, int chunk_rows,
                      uint32_t epoch, uint32_t* status, int sm_limit, cudaStream_t stream) {
  if (M <= 0) return;
  if (chunk_rows % TP_BM != 0 || N % 8 != 0 || N > TP_THREADS * 6 * 8)
    throw std::runtime_error("gemm_rs_add_norm: chunk_rows must be a multiple of 128 and N <= 9216, N % 8 == 0");
  TpGemmParams p{};
  fill_common(p, M, N, K, b.world, b.rank, chunk_rows, epoch, status, false);
  // the grouped raster must see `padded` m-blocks
  const int padded_m = p.tp * p.blocks_per_chunk;
  const int real_num_m = p.num_m;
  for (int i = 0; i < b.world; ++i) {
    p.stage_peer[i] = b.stage[i];
    p.rs_flag_peer[i] = b.rs_flags[i];
    p.xg_peer[i] = b.xg[i];
    p.gathered_flag_peer[i] = b.gathered_flags[i];
  }
  p.stage_local = b.stage[b.rank];
  p.rs_flags_local = b.rs_flags[b.rank];
  p.owner_done = b.owner_done;
  p.pipelined = (tp_pipeline_enabled() && b.group_done != nullptr && p.blocks_per_chunk <= b.max_groups) ? 1 : 0;
  p.max_groups = b.max_groups;
  p.group_done = b.group_done;
  for (int i = 0; i < b.world; ++i) p.group_flag_peer[i] = b.group_flags[i];
  p.group_flags_local = b.group_flags[b.rank];
  const bool nvls = p.pipelined && tp_nvls_enabled() && b.stage_mc != nullptr && b.xg_mc != nullptr;
  p.stage_mc = nvls ? b.stage_mc : nullptr;
  p.xg_mc = nvls ? b.xg_mc : nullptr;
  p.stage_rw = b.stage[b.rank];
  p.residual = reinterpret_cast<__nv_bfloat16*>(residual);
  p.norm_w = reinterpret_cast<const __nv_bfloat16*>(norm_w);
  p.eps = eps;
  (void)padded_m;
  (void)real_num_m;
  const CUtensorMap ta = make_tmap_bf16_2d(x, M, K, ldx, TP_BM, TP_BK);
  const CUtensorMap tb = make_tmap_bf16_2d(w, N, K, ldw, TP_BN, TP_BK);
  const int sms = sm_limit > 0 ? sm_limit : gemm_num_sms();
  // Every CTA takes part in the flag exchange of phase 2, and a flag is raised only when ALL tiles of a rank are
  // delivered, so every CTA must get an SM without another CTA of this grid having to finish first.  The grid is
  // therefore at most one CTA per SM of the stream's SM set (the green context's, if any).  Kernels of other
  // streams can delay a CTA's start (they end without waiting for this kernel) but not prevent it; the waits of
  // phase 2 are bounded and report through the status word if that delay ever exceeded the limit.
  if (p.pipelined && p.stage_mc != nullptr) {
    auto kern = gemm_tp_kernel<MODE_RS, true, true>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tp_smem_bytes());
    kern<<<std::min(p.total_tiles, sms), TP_THREADS_RS, tp_smem_bytes(), stream>>>(ta, tb, p);
  } else if (p.pipelined) {
    auto kern = gemm_tp_kernel<MODE_RS, true, false>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tp_smem_bytes());
    kern<<<std::min(p.total_tiles, sms), TP_THREADS_RS, tp_smem_bytes(), stream>>>(ta, tb, p);
  } else {
    auto kern = gemm_tp_kernel<MODE_RS, false>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tp_smem_bytes());
    kern<<<std::min(p.total_tiles, sms), TP_THREADS, tp_smem_bytes(), stream>>>(ta, tb, p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("gemm_rs_add_norm launch: ") + cudaGetErrorString(e));
}

void gemm_after_gather(const void* xg_local, const void* w, void* c, int M, int N, int K, long long ldw,
                       long long ldc, const TpBuffers& b, int chunk_rows, uint32_t epoch, uint32_t* status,
                       int sm_limit, cudaStream_t stream, bool swiglu) {
  if (M <= 0) return;
  TpGemmParams p{};
  fill_common(p, M, N, K, b.world, b.rank, chunk_rows, epoch, status, true);
  p.C = reinterpret_cast<__nv_bfloat16*>(c);
  p.ldc = ldc;
  p.gathered_flags = b.gathered_flags[b.rank];
  const CUtensorMap ta = make_tmap_bf16_2d(xg_local, M, K, K, TP_BM, TP_BK);
  const int sms = sm_limit > 0 ? sm_limit : gemm_num_sms();
  if (swiglu) {
    // w = [gate; up] ([N, K], N = 2 x width); c is [M, N / 2]
    if (N % 256 != 0 || ldc % 8 != 0) throw std::runtime_error("gemm_after_gather: SwiGLU needs N % 256 == 0");
    const int width = N / 2;
    p.N = width;
    p.up_row0 = width;
    p.num_n = width / (TP_BN / 2);
    p.total_tiles = p.tp * p.blocks_per_chunk * p.num_n;
    const CUtensorMap tb = make_tmap_bf16_2d(w, N, K, ldw, TP_BN / 2, TP_BK);
    auto kern = gemm_tp_kernel<MODE_AG_SWIGLU>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tp_smem_bytes());
    kern<<<std::min(p.total_tiles, sms), TP_THREADS, tp_smem_bytes(), stream>>>(ta, tb, p);
    cudaError_t e2 = cudaGetLastError();
    if (e2 != cudaSuccess)
      throw std::runtime_error(std::string("gemm_after_gather (SwiGLU) launch: ") + cudaGetErrorString(e2));
    return;
  }
  const CUtensorMap tb = make_tmap_bf16_2d(w, N, K, ldw, TP_BN, TP_BK);
  auto kern = gemm_tp_kernel<MODE_AG>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tp_smem_bytes());
  kern<<<std::min(p.total_tiles, sms), TP_THREADS, tp_smem_bytes(), stream>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("gemm_after_gather launch: ") + cudaGetErrorString(e));
}

}  // namespace fc
