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
// Split-K inside a thread-block cluster (`cluster` > 0; opt-in, see cluster_splitk_enabled): the K splits of one row
// tile are the CTAs of one cluster (cluster dims (1, splits, 1)).  When the mainloops are done the CTAs exchange
// their fp32 accumulators through distributed shared memory, reduce-scatter fashion: the token columns are dealt
// out in chunks of 32, every CTA sends each chunk to the CTA that owns it (st.shared::cluster into the owner's idle
// operand stages) and sums the chunks it owns, then applies bias / activation and writes bf16.  No partial sums go
// to global memory and no second kernel reads them back.  With `swiglu` the two 128-row halves of a tile are the
// gate rows and the matching up rows of a [gate; up] weight, and the epilogue writes silu(gate) * up.
// Every CTA loads its own operand tiles (no multicast); the cluster is only used for the exchange.
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
#include <cstdio>
#include <cstdlib>
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
  int cluster;            // > 0: the splits are the CTAs of a cluster and reduce through shared memory
  int swiglu;             // cluster mode only: tile = 128 gate rows + the matching 128 up rows, out [Mtok, Nw / 2]
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
  // first W row of the two 128-row halves of this CTA's tile
  const int w_row0 = p.swiglu ? tile * 128 : tile * ROWS;
  const int w_row1 = p.swiglu ? p.Nw / 2 + tile * 128 : tile * ROWS + 128;
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
        tma_load_2d(sa, &tma_w, &full_bar[s], (kb0 + s) * SK_BK, w_row0);
        if constexpr (MT == 2)
          tma_load_2d(sa + L::A_BYTES / 2, &tma_w, &full_bar[s], (kb0 + s) * SK_BK, w_row1);
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
        tma_load_2d(sa, &tma_w, &full_bar[stage], kb * SK_BK, w_row0);
        if constexpr (MT == 2)
          tma_load_2d(sa + L::A_BYTES / 2, &tma_w, &full_bar[stage], kb * SK_BK, w_row1);
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
    if (p.cluster > 0) {
      // the accumulators are exchanged and reduced after the role branches, by all CTAs of the cluster together
      if (*s_abort || !mbar_wait(acc_full, 0, p.status, ST_TIMEOUT_ACC_FULL)) *s_abort = 1;
      tc_fence_after();
    } else if (!*s_abort && mbar_wait(acc_full, 0, p.status, ST_TIMEOUT_ACC_FULL)) {
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
  if (p.cluster > 0) {
    // ------------------------------------------------- split-K reduction through distributed shared memory
    // Every thread of every CTA of the cluster comes through here, whatever happened in its role branch (the two
    // cluster barriers below count all of them).  Chunk c (tokens 32 c ... 32 c + 31) belongs to CTA c % S.
    const int S = int(cluster_nctarank()), me = int(cluster_ctarank());
    constexpr int CHUNKS = BN / 32;
    const int cl_max = (CHUNKS + S - 1) / S;                 // chunks a CTA can own
    constexpr uint32_t SLOT_BYTES = 8 * 128 * 16;            // one chunk of one 128-row half: [8 x float4][128 rows]
    const uint32_t recv0 = smem_u32(smem);                   // the operand stages are idle once the MMAs are done
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;
    const uint32_t t_row = tmem_base + (uint32_t(lane_group * 32) << 16);
    __syncwarp();
    if (S > 1) cluster_sync();                               // 1: every CTA's mainloop is over, its stages are free
    if (warp >= 2 && S > 1 && !*s_abort) {
#pragma unroll 1
      for (int c = 0; c < CHUNKS; ++c) {
        const int owner = c % S;
        if (owner == me) continue;
        const int src = me < owner ? me : me - 1;            // my index among the owner's S - 1 senders
#pragma unroll 1
        for (int mt = 0; mt < MT; ++mt) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + uint32_t(mt * BN + c * 32), r);
          tmem_ld_wait();
          const uint32_t slot = uint32_t((src * MT + mt) * cl_max + c / S);
          const uint32_t dst = cluster_map_shared(recv0 + slot * SLOT_BYTES, uint32_t(owner)) + uint32_t(row) * 16u;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            st_cluster_f32x4(dst + uint32_t(j) * 128u * 16u, __uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                             __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        }
      }
    }
    __syncwarp();
    if (S > 1) cluster_sync();                               // 2: all chunks have landed at their owners
    if (warp >= 2 && !*s_abort) {
      const int width = p.swiglu ? p.Nw / 2 : p.Nw;          // output columns
#pragma unroll 1
      for (int c = me; c < CHUNKS; c += S) {
        if (c * 32 >= p.Mtok) break;
        float acc[MT][32];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + uint32_t(mt * BN + c * 32), r);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 32; ++t) acc[mt][t] = __uint_as_float(r[t]);
#pragma unroll 1
          for (int src = 0; src < S - 1; ++src) {
            const uint8_t* slot = smem + size_t((src * MT + mt) * cl_max + c / S) * SLOT_BYTES + size_t(row) * 16;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 v = *reinterpret_cast<const float4*>(slot + size_t(j) * 128 * 16);
              acc[mt][4 * j] += v.x;
              acc[mt][4 * j + 1] += v.y;
              acc[mt][4 * j + 2] += v.z;
              acc[mt][4 * j + 3] += v.w;
            }
          }
        }
        if (p.swiglu) {
          if constexpr (MT == 2) {
            const int n = tile * 128 + row;
            if (n < width) {
#pragma unroll
              for (int t = 0; t < 32; ++t) {
                const int tok = c * 32 + t;
                if (tok < p.Mtok) {
                  // gate and up rounded to bf16 first: the values a separate SwiGLU kernel would read
                  const float g = __bfloat162float(__float2bfloat16(acc[0][t]));
                  const float u = __bfloat162float(__float2bfloat16(acc[1][t]));
                  p.out[(long long)tok * p.ldc + n] = __float2bfloat16(g / (1.f + __expf(-g)) * u);
                }
              }
            }
          }
        } else {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const int n = tile * ROWS + mt * 128 + row;
            if (n < width) {
              const float bi = p.bias != nullptr ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll
              for (int t = 0; t < 32; ++t) {
                const int tok = c * 32 + t;
                if (tok < p.Mtok)
                  p.out[(long long)tok * p.ldc + n] = __float2bfloat16(sk_act(acc[mt][t] + bi, p.act));
              }
            }
          }
        }
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

static bool skinny_debug() {
  static const bool on = std::getenv("FC_SKINNY_DEBUG") != nullptr;
  return on;
}
static int g_cluster_splitk = -1;
bool cluster_splitk_enabled() {
  if (g_cluster_splitk < 0) {
    // off unless asked for.  Measured on B200 (128 tokens): 0.161 ms against 0.088 ms for the 24576 x 4096 gate/up
    // projection, 0.049 against 0.039 ms for qkv, 0.60 against 0.40 ms for the LM head.  Clusters of 2 / 3 / 4 CTAs
    // of this kernel (one CTA per SM) fit 74 / 45 / 33 times on the 148 SMs, so the grid loses SMs and whole waves
    // to the cluster granularity, and the exchange moves the same bytes between SMs that the partial sums move
    // through L2.
    const char* e = std::getenv("FC_CLUSTER_SPLITK");
    g_cluster_splitk = (e != nullptr && std::string(e) == "1") ? 1 : 0;
  }
  return g_cluster_splitk == 1;
}
void set_cluster_splitk(bool on) { g_cluster_splitk = on ? 1 : 0; }

// How many clusters of `cluster_y` CTAs of this kernel the device holds at once (0: such clusters cannot be placed).
template <int BN, int STAGES, int ROWS>
static int skinny_max_clusters(int cluster_y) {
  using L = SkinnySmem<BN, STAGES, ROWS>;
  static int cache[64][9];
  static bool init = false;
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!init) {
    for (auto& row : cache)
      for (int& v : row) v = -1;
    init = true;
  }
  if (cluster_y < 1 || cluster_y > 8) return 0;
  if (cache[dev][cluster_y] >= 0) return cache[dev][cluster_y];
  auto kern = gemm_skinny_kernel<BN, STAGES, ROWS>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(1, cluster_y, 1);
  cfg.blockDim = dim3(SK_THREADS);
  cfg.dynamicSmemBytes = L::TOTAL;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = cluster_y;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  cache[dev][cluster_y] = n;
  return n;
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
  cudaError_t e = p.cluster > 0
      ? launch_pdl_cluster(PDL_SKINNY_GEMM, kern, dim3(tiles, p.splits), dim3(SK_THREADS), L::TOTAL, stream,
                           unsigned(p.splits), tw, tx, p)
      : launch_pdl(PDL_SKINNY_GEMM, kern, dim3(tiles, p.splits), dim3(SK_THREADS), L::TOTAL, stream, tw, tx, p);
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

// Cluster form: K splits = CTAs of a cluster.  S must leave room for the exchange in the operand stages
// ((S - 1) x halves x owned chunks x 16 KiB) and clusters of S must be placeable; cost as above with waves counted in
// clusters.  Returns 0 when no S (not even 1) fits.
template <int BN, int STAGES, int ROWS>
static int skinny_pick_cluster(int tiles, int num_kb, int sms_cap) {
  using L = SkinnySmem<BN, STAGES, ROWS>;
  constexpr int MT = ROWS / 128, CHUNKS = BN / 32;
  int best = 0;
  double best_cost = 1e30;
  for (int s = 1; s <= 8 && s <= CHUNKS; ++s) {
    if (s > 1 && num_kb / s < 2) break;
    if ((num_kb + (num_kb + s - 1) / s - 1) / ((num_kb + s - 1) / s) != s) continue;   // every CTA must get K blocks
    const int cl_max = (CHUNKS + s - 1) / s;
    if ((s - 1) * MT * cl_max * (8 * 128 * 16) > L::BAR_OFF) continue;
    int active = skinny_max_clusters<BN, STAGES, ROWS>(s);
    if (sms_cap > 0) active = std::min(active, sms_cap / s);
    if (active <= 0) continue;
    const int waves = (tiles + active - 1) / active;
    const int kb = (num_kb + s - 1) / s;
    const double cost = waves * (kb + 6.0) + 0.7 * (s - 1);      // the exchange grows a little with the cluster
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
                     int splits_request, bool finalize, cudaStream_t stream, const SkinnyFused* fused, int flags) {
  const int sms = sm_limit > 0 ? sm_limit : gemm_num_sms();
  const int num_kb = (K + SK_BK - 1) / SK_BK;
  const bool swiglu = (flags & SK_SWIGLU) != 0;
  if (swiglu && (N % 256 != 0 || fused != nullptr || bias != nullptr)) return 0;
  // 128-row tiles when 256-row tiles would cover less than half of the SMs: the same SM count is then reached
  // with half the K splits, i.e. half the partial-sum traffic.  (SwiGLU tiles are 128 gate + 128 up rows.)
  const bool small_rows = !swiglu && (N + SK_BM - 1) / SK_BM <= sms / 2;
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
  // ---- the cluster form, where allowed: the splits become the CTAs of a cluster and nothing is left for a consumer
  int cluster = 0;
  const bool want_cluster = !fuse && splits_request <= 0 && (flags & SK_NO_CLUSTER) == 0 && cluster_splitk_enabled();
  if (want_cluster || swiglu) {
    const int cap = sm_limit > 0 ? sm_limit : 0;
    int s_c = 0;
    if (M <= 32) s_c = small_rows ? skinny_pick_cluster<32, 8, 128>(tiles, num_kb, cap) : skinny_pick_cluster<32, 6, 256>(tiles, num_kb, cap);
    else if (M <= 64) s_c = small_rows ? skinny_pick_cluster<64, 7, 128>(tiles, num_kb, cap) : skinny_pick_cluster<64, 5, 256>(tiles, num_kb, cap);
    else if (M <= 128) s_c = small_rows ? skinny_pick_cluster<128, 6, 128>(tiles, num_kb, cap) : skinny_pick_cluster<128, 4, 256>(tiles, num_kb, cap);
    else s_c = small_rows ? skinny_pick_cluster<256, 4, 128>(tiles, num_kb, cap) : skinny_pick_cluster<256, 3, 256>(tiles, num_kb, cap);
    if (s_c > 0) {
      cluster = 1;
      splits = s_c;
    } else if (swiglu) {
      return 0;
    }
  }
  int kb_per = (num_kb + splits - 1) / splits;
  if (!cluster) splits = (num_kb + kb_per - 1) / kb_per;      // (the cluster sizes were chosen so that this holds)
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
  p.cluster = cluster;
  p.swiglu = swiglu ? 1 : 0;
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
  if (skinny_debug()) {
    int act8[9] = {0};
    for (int s_ = 1; s_ <= 8; ++s_) act8[s_] = (M <= 128 && M > 64) ? (small_rows ? skinny_max_clusters<128, 6, 128>(s_) : skinny_max_clusters<128, 4, 256>(s_)) : -1;
    fprintf(stderr, "[skinny] M=%d N=%d K=%d rows=%d tiles=%d cluster=%d splits=%d kb_per=%d active(1..8)=%d %d %d %d %d %d %d %d\n",
            M, N, K, rows, tiles, cluster, splits, kb_per, act8[1], act8[2], act8[3], act8[4], act8[5], act8[6], act8[7], act8[8]);
  }
  if (cluster) return 1;               // finished bf16 result in `c`
  if (splits > 1 && finalize && !fuse) {
    const long long total = (long long)M * (N / 4);
    const int blocks = (int)std::min<long long>((total + 255) / 256, 2048);
    launch_pdl(PDL_FINALIZE, skinny_finalize_kernel, dim3(blocks), dim3(256), 0, stream, (const float*)ws.scratch, p.bias, p.out, M,
               N, ldc, splits, act);
  }
  return splits;
}

}  // namespace fc
