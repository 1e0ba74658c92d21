// Tensor-parallel communication fused with the residual add and RMSNorm.
//
// allreduce_add_rmsnorm (decode-size inputs, "one shot"): every rank holds a bf16
// partial [T, H] in a symmetric buffer (the row-parallel GEMM wrote it there).
// One kernel, one CTA per token row:
//   1. flag exchange with the same CTA on every peer ("my partial is complete");
//      the stores are st.release.sys to the peers' signal pads, the wait is a
//      bounded ld.acquire.sys spin that reports ST_TIMEOUT_PEER instead of hanging
//   2. sum of the row over all ranks, read either with plain peer loads in rank
//      order (bit-identical on every rank) or with one multimem.ld_reduce per
//      16 bytes through the NVSwitch multicast address
//   3. + residual (updated in place), RMSNorm, normalised row written locally
// The buffers are used in alternation (two per rank) and the per-CTA epoch lives
// in device memory, so the kernel can be replayed from a CUDA graph: a rank can
// only overwrite a buffer after it has passed the next flag exchange, which every
// peer joins only after it finished reading that buffer.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

#include "comm.h"
#include "comm_dev.cuh"
#include "launch.h"
#include "ptx.cuh"
#include "sample.cuh"

namespace fc {

using bf16 = __nv_bfloat16;

// Exchange "arrived" flags between CTA `slot` of all ranks.  Returns false on timeout.
__device__ __forceinline__ bool peer_barrier(const CommPeers& peers, int slot, uint32_t epoch, uint32_t* status) {
  const int tid = threadIdx.x;
  __shared__ int s_ok;
  if (tid == 0) s_ok = 1;
  __syncthreads();
  if (tid < peers.world && !peer_flag_exchange(peers, slot, epoch, tid, status)) s_ok = 0;
  __syncthreads();
  return s_ok != 0;
}

constexpr int AR_THREADS = 256;
constexpr int AR_MAX_CHUNKS = 4;      // H <= 256 * 4 * 8 = 8192

// MODE 0: peer loads after the flag exchange; 1: multimem.ld_reduce after it; 2: peer STORES before it ("push":
// one row per CTA; the CTA finishes its row, stores it into its slot of every peer's staging buffer, then the
// flag exchange publishes those stores, then every rank sums the `world` slots of its OWN buffer in rank order,
// its own contribution from registers).  The push form takes the NVLink round trip of the loads out of the
// critical path: the stores are posted and travel while the CTA is already waiting for the flags.
constexpr int AR_PULL = 0, AR_MULTIMEM = 1, AR_PUSH = 2, AR_TWOSHOT = 3;

__device__ __forceinline__ void multimem_st_16(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_peer_16(void* p, const uint4& v) {
  asm volatile("st.global.relaxed.sys.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(AR_THREADS)
allreduce_add_rmsnorm_kernel(CommPeers peers, int buf, const bf16* __restrict__ mc_in, bf16* __restrict__ residual,
                             const bf16* __restrict__ weight, bf16* __restrict__ out, int T, int H, float eps,
                             uint32_t* __restrict__ epochs, uint32_t* status, const float* __restrict__ partial,
                             int splits, long long split_stride, const bf16* __restrict__ bias) {
  __shared__ float red[32];
  __shared__ uint32_t s_epoch;
  pdl_launch_dependents();
  pdl_wait();                            // the GEMM that filled the staging buffer, the previous epoch counters
  uint4 mine[AR_MAX_CHUNKS];             // AR_PUSH: this rank's finished row, 16 bytes per chunk and thread
  if (MODE == AR_PUSH) {
    // grid == T: CTA b owns token row b.  Slot `rank` of every staging buffer receives this rank's row.
    const int row = blockIdx.x;
    const size_t slot_off = ((size_t)peers.rank * peers.slot_rows + row) * H;
    const int chunks0 = H >> 3;
#pragma unroll
    for (int c = 0; c < AR_MAX_CHUNKS; ++c) {
      const int idx = threadIdx.x + c * AR_THREADS;
      if (idx < chunks0) {
        if (partial != nullptr) {
          const size_t off = (size_t)row * H + (size_t)idx * 8;
          float acc[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll 4
          for (int s = 0; s < splits; ++s) {
            const float4* ps = reinterpret_cast<const float4*>(partial + (size_t)s * split_stride + off);
            const float4 a = __ldcg(ps), b = __ldcg(ps + 1);
            acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
            acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
          }
          if (bias != nullptr) {
            float bb[8];
            unpack8f(*reinterpret_cast<const uint4*>(bias + (size_t)idx * 8), bb);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += bb[i];
          }
          mine[c] = pack8f(acc);
        } else {
          // the GEMM wrote finished bf16 rows into this rank's own slot of its own buffer
          mine[c] = *reinterpret_cast<const uint4*>(peers.data[buf][peers.rank] + slot_off + (size_t)idx * 8);
        }
#pragma unroll
        for (int d = 0; d < COMM_MAX_WORLD; ++d)
          if (d < peers.world && d != peers.rank) st_peer_16(peers.data[buf][d] + slot_off + (size_t)idx * 8, mine[c]);
      }
    }
    __syncthreads();
  } else if (partial != nullptr) {
    // the GEMM left split-K partial sums [splits, T, H] in local scratch: finish this CTA's rows into this
    // rank's staging buffer first (what the GEMM's finalize kernel would have done), then join the exchange
    bf16* mine = peers.data[buf][peers.rank];
    const int chunks0 = H >> 3;
    for (int row = blockIdx.x; row < T; row += gridDim.x) {
      for (int idx = threadIdx.x; idx < chunks0; idx += AR_THREADS) {
        const size_t off = (size_t)row * H + (size_t)idx * 8;
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll 4
        for (int s = 0; s < splits; ++s) {
          const float4* ps = reinterpret_cast<const float4*>(partial + (size_t)s * split_stride + off);
          const float4 a = __ldcg(ps), b = __ldcg(ps + 1);
          acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
          acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
        }
        if (bias != nullptr) {
          float bb[8];
          unpack8f(*reinterpret_cast<const uint4*>(bias + (size_t)idx * 8), bb);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += bb[i];
        }
        *reinterpret_cast<uint4*>(mine + off) = pack8f(acc);
      }
    }
    __syncthreads();
  }
  const int slot = blockIdx.x;
  if (threadIdx.x == 0) s_epoch = epochs[slot] + 1;
  __syncthreads();
  const uint32_t epoch = s_epoch;
  bool ok = peer_barrier(peers, slot, epoch, status);
  if (MODE == AR_TWOSHOT) {
    // grid == T: CTA b owns token row b; rank (b % world) reduces it inside the switch and publishes the sum.
    // Every rank joins the second exchange, also after a first one that ran out (the peers must not wait for it).
    const int row = blockIdx.x;
    if (ok && row % peers.world == peers.rank) {
      const int chunks0 = H >> 3;
      for (int idx = threadIdx.x; idx < chunks0; idx += AR_THREADS) {
        const size_t off = (size_t)row * H + (size_t)idx * 8;
        const uint4 sum = multimem_ld_reduce_bf16x8(mc_in + off);
        multimem_st_16(const_cast<bf16*>(mc_in) + (size_t)peers.reduced_row0 * H + off, sum);
      }
      __threadfence_system();
    }
    __syncthreads();
    const bool ok2 = peer_barrier(peers, slot, epoch + 1, status);
    ok = ok && ok2;
    if (threadIdx.x == 0) epochs[slot] = epoch + 1;
  } else {
    if (threadIdx.x == 0) epochs[slot] = epoch;
  }
  if (!ok) return;                       // the host reads the status word and raises

  const int chunks = H >> 3;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const size_t base = (size_t)row * H;
    float v[AR_MAX_CHUNKS][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < AR_MAX_CHUNKS; ++c) {
      const int idx = threadIdx.x + c * AR_THREADS;
      if (idx < chunks) {
        const size_t off = base + (size_t)idx * 8;
        float acc[8];
        if (MODE == AR_MULTIMEM) {
          unpack8f(multimem_ld_reduce_bf16x8(mc_in + off), acc);
        } else if (MODE == AR_TWOSHOT) {
          // the row's sum over all ranks, published by its owner into this rank's own buffer
          unpack8f(ld_peer_16(peers.data[buf][peers.rank] + (size_t)peers.reduced_row0 * H + off), acc);
        } else if (MODE == AR_PUSH) {
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = 0.f;
          // the peers' rows are in this rank's own buffer now (the flag exchange made their stores visible)
          uint4 raw[COMM_MAX_WORLD];
          const bf16* here = peers.data[buf][peers.rank];
#pragma unroll
          for (int p = 0; p < COMM_MAX_WORLD; ++p)
            if (p < peers.world)
              raw[p] = p == peers.rank ? mine[c]
                                       : ld_peer_16(here + ((size_t)p * peers.slot_rows + row) * H + (size_t)idx * 8);
#pragma unroll
          for (int p = 0; p < COMM_MAX_WORLD; ++p) {
            if (p < peers.world) {
              float f[8];
              unpack8f(raw[p], f);
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[i] += f[i];
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = 0.f;
          // all peers' pieces are requested before the first is used (one NVLink round trip, not `world`)
          uint4 raw[COMM_MAX_WORLD];
#pragma unroll
          for (int p = 0; p < COMM_MAX_WORLD; ++p)
            if (p < peers.world) raw[p] = ld_peer_16(peers.data[buf][p] + off);
#pragma unroll
          for (int p = 0; p < COMM_MAX_WORLD; ++p) {
            if (p < peers.world) {
              float f[8];
              unpack8f(raw[p], f);
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[i] += f[i];
            }
          }
        }
        float r[8];
        unpack8f(*reinterpret_cast<const uint4*>(residual + off), r);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += r[i];
        const uint4 s = pack8f(acc);
        *reinterpret_cast<uint4*>(residual + off) = s;
        unpack8f(s, v[c]);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[c][i] * v[c][i];
      }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < AR_THREADS / 32; ++w) tot += red[w];
    __syncthreads();
    const float inv = rsqrtf(tot / float(H) + eps);
#pragma unroll
    for (int c = 0; c < AR_MAX_CHUNKS; ++c) {
      const int idx = threadIdx.x + c * AR_THREADS;
      if (idx < chunks) {
        float g[8], o[8];
        unpack8f(*reinterpret_cast<const uint4*>(weight + (size_t)idx * 8), g);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __bfloat162float(__float2bfloat16(v[c][i] * inv)) * g[i];
        *reinterpret_cast<uint4*>(out + base + (size_t)idx * 8) = pack8f(o);
      }
    }
  }
}

void launch_allreduce_add_rmsnorm(const CommPeers& peers, int buf, const void* mc_in, void* residual,
                                  const void* weight, void* out, int T, int H, float eps, uint32_t* epochs,
                                  uint32_t* status, bool use_multimem, cudaStream_t stream, const float* partial,
                                  int splits, long long split_stride, const void* bias) {
  if (T == 0) return;
  if (H % 8 != 0 || H > AR_THREADS * AR_MAX_CHUNKS * 8) throw std::runtime_error("allreduce: unsupported hidden size");
  // CTA b exchanges flags only with CTA b of the peers (no CTA waits for another CTA of its own grid), and CTAs
  // are dispatched in index order on every rank, so the lowest unfinished slot is resident everywhere and the
  // exchange makes progress even while kernels of other streams hold SMs.  The grid is still kept within what
  // one GPU holds at once (COMM_MAX_SLOTS CTAs, several per SM) so that no slot waits for a whole wave.
  const int grid = T < COMM_MAX_SLOTS ? T : COMM_MAX_SLOTS;
  cudaError_t e;
  if (peers.reduced_row0 > 0 && mc_in != nullptr) {
    if (T > peers.reduced_row0 || T > COMM_MAX_SLOTS)
      throw std::runtime_error("allreduce (two-shot form): more token rows than the staging buffer holds");
    e = launch_pdl(PDL_ALLREDUCE, allreduce_add_rmsnorm_kernel<AR_TWOSHOT>, dim3(T), dim3(AR_THREADS), 0, stream, peers, buf,
                   (const bf16*)mc_in, (bf16*)residual, (const bf16*)weight, (bf16*)out, T, H, eps, epochs, status,
                   partial, splits, split_stride, (const bf16*)bias);
  } else if (peers.slot_rows > 0) {
    if (T > peers.slot_rows || T > COMM_MAX_SLOTS)
      throw std::runtime_error("allreduce (push form): more token rows than a staging slot holds");
    e = launch_pdl(PDL_ALLREDUCE, allreduce_add_rmsnorm_kernel<AR_PUSH>, dim3(T), dim3(AR_THREADS), 0, stream, peers, buf,
                   (const bf16*)nullptr, (bf16*)residual, (const bf16*)weight, (bf16*)out, T, H, eps, epochs, status,
                   partial, splits, split_stride, (const bf16*)bias);
  } else if (use_multimem && mc_in != nullptr)
    e = launch_pdl(PDL_ALLREDUCE, allreduce_add_rmsnorm_kernel<AR_MULTIMEM>, dim3(grid), dim3(AR_THREADS), 0, stream, peers, buf,
                   (const bf16*)mc_in, (bf16*)residual, (const bf16*)weight, (bf16*)out, T, H, eps, epochs, status,
                   partial, splits, split_stride, (const bf16*)bias);
  else
    e = launch_pdl(PDL_ALLREDUCE, allreduce_add_rmsnorm_kernel<AR_PULL>, dim3(grid), dim3(AR_THREADS), 0, stream, peers, buf,
                   (const bf16*)nullptr, (bf16*)residual, (const bf16*)weight, (bf16*)out, T, H, eps, epochs, status,
                   partial, splits, split_stride, (const bf16*)bias);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("allreduce launch: ") + cudaGetErrorString(e));
}

// ---------------------------------------------------------------- sampling over vocabulary shards
// Every rank holds the logits of its vocabulary shard.  One CTA per request finds the shard's best candidate
// (see sample.cuh), stores it as one 8-byte cell into every rank's candidate table, exchanges flags exactly like
// the all-reduce above and picks the winner of the `world` candidates.  All ranks see the same candidates, so
// they all return the same token: no gather of the logits, no broadcast of the tokens.  The table has two
// halves used by even and odd epochs, so a rank that is one exchange ahead never overwrites a cell a peer
// still has to read.
__device__ __forceinline__ void st_relaxed_sys_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_relaxed_sys_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(1024)
sample_exchange_kernel(CommPeers peers, SamplePeers cand, const bf16* __restrict__ logits,
                       const float* __restrict__ temps, long long* __restrict__ out, int V, long long ld,
                       uint32_t seed, int vocab_offset, int v_limit, uint32_t* __restrict__ epochs,
                       uint32_t* status) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ uint64_t s_cand[COMM_MAX_WORLD];
  __shared__ uint64_t s_mine;
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;                       // also the flag slot
  float best;
  int best_i;
  sample_row_best(logits + (long long)b * ld, V, vocab_offset, v_limit, temps[b], sample_row_seed(seed, b), s_val,
                  s_idx, best, best_i);
  if (threadIdx.x == 0) {
    s_mine = (uint64_t(__float_as_uint(best)) << 32) | uint64_t(uint32_t(best_i));
    s_epoch = epochs[b] + 1;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int tid = threadIdx.x;
  if (tid < peers.world) {
    const size_t half = size_t(epoch & 1u) * COMM_MAX_SLOTS;
    // candidate first, then the flag, both by this thread: the release orders them for the peer
    st_relaxed_sys_u64(cand.cells[tid] + (half + b) * COMM_MAX_WORLD + peers.rank, s_mine);
    st_release_sys(peers.flags[tid] + (size_t)b * COMM_MAX_WORLD + peers.rank, epoch);
    const uint32_t* mine = peers.flags[peers.rank] + (size_t)b * COMM_MAX_WORLD + tid;
    bool got = false;
    const uint64_t t0 = global_timer_ns();
    uint64_t limit = FC_PEER_WAIT_LIMIT_NS;
    for (uint32_t i = 0; i < FC_PEER_SPIN_LIMIT; ++i) {
      if (int32_t(ld_acquire_sys(mine) - epoch) >= 0) {
        got = true;
        break;
      }
      __nanosleep(20);
      if ((i & 255u) == 255u) {
        if (i == 255u) limit = peer_wait_limit_ns(status);
        if (global_timer_ns() - t0 > limit) break;
      }
    }
    if (got) {
      s_cand[tid] = ld_relaxed_sys_u64(cand.cells[peers.rank] + (half + b) * COMM_MAX_WORLD + tid);
    } else {
      report(status, ST_TIMEOUT_PEER);
      s_ok = 0;
    }
  }
  __syncthreads();
  if (tid == 0) {
    epochs[b] = epoch;
    if (s_ok) {
      best = -INFINITY;
      best_i = 0x7fffffff;
      for (int p = 0; p < peers.world; ++p) {
        const float v = __uint_as_float(uint32_t(s_cand[p] >> 32));
        const int i = int(uint32_t(s_cand[p]));
        if (sample_better(v, i, best, best_i)) {
          best = v;
          best_i = i;
        }
      }
    }
    out[b] = best_i;                 // after a timeout: this shard's own candidate; the host raises on the status
    if (b == 0) out[gridDim.x] = (long long)(*reinterpret_cast<const volatile uint32_t*>(status) & ST_CODE_MASK);
  }
}

void launch_sample_exchange(const CommPeers& peers, const SamplePeers& cand, const void* logits, const void* temps,
                            void* out, int B, int V, long long ld, uint32_t seed, int vocab_offset, int v_limit,
                            uint32_t* epochs, uint32_t* status, cudaStream_t stream) {
  if (B == 0) return;
  if (B > COMM_MAX_SLOTS) throw std::runtime_error("sample exchange: more requests than flag slots");
  cudaError_t e = launch_pdl(PDL_SAMPLE, sample_exchange_kernel, dim3(B), dim3(1024), 0, stream, peers, cand,
                             (const bf16*)logits, (const float*)temps, (long long*)out, V, ld, seed, vocab_offset,
                             v_limit, epochs, status);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("sample exchange launch: ") + cudaGetErrorString(e));
}

}  // namespace fc

namespace fc {

__global__ void wait_gathered_kernel(const uint32_t* flags, int world, uint32_t epoch, uint32_t* status) {
  if (threadIdx.x < world) {
    const uint64_t t0 = global_timer_ns();
    const uint64_t limit = peer_wait_limit_ns(status);
    bool got = false;
    for (uint32_t i = 0; i < FC_PEER_SPIN_LIMIT; ++i) {
      if (int32_t(ld_acquire_sys(flags + threadIdx.x) - epoch) >= 0) {
        got = true;
        break;
      }
      __nanosleep(40);
      if ((i & 255u) == 255u && global_timer_ns() - t0 > limit) break;
    }
    if (!got) report(status, ST_TIMEOUT_PEER);
  }
}

void wait_gathered(const TpBuffers& b, uint32_t epoch, uint32_t* status, cudaStream_t stream) {
  wait_gathered_kernel<<<1, 32, 0, stream>>>(b.gathered_flags[b.rank], b.world, epoch, status);
}

}  // namespace fc
