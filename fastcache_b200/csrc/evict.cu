// KV eviction in the paged pool: key-norm scoring, per-head top-k selection and
// stable in-place compaction.
//
// Pool layout [L, 2, num_blocks, Hkv, block_size, D] bf16 (rows of one head contiguous in a block).  Scores are fp32
// [n_seq, L, Hkv, s_stride], higher = keep (+inf = always keep).
//
// select_compact: one CTA per (kv head, layer, request).  The scores of the
// request are turned into order-preserving 32-bit keys in shared memory, the
// k-th largest key is found with a 4-pass radix select, and the kept rows
// (ties resolved toward later rows) are moved to the front of the request's rows
// in ascending order.  A destination index never exceeds its source index, and
// each 128-row chunk is read completely into registers before it is written, so
// the compaction is safe in place.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

#include "kernels.h"
#include "ptx.cuh"

namespace fc {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// scores[seq, layer, h, tok] = sign * ||K[tok, h, :]||      (mode 0: per head)
//                            = mean_h ||K[tok, h, :]||       (mode 1: shared by heads, largest kept)
constexpr int KN_ROWS = 32;

__global__ void __launch_bounds__(256)
knorm_score_kernel(const bf16* __restrict__ pool, const int* __restrict__ block_tables,
                   const int* __restrict__ kv_lens, float* __restrict__ scores, int L, int num_blocks,
                   int block_size, int Hkv, int D, int max_blocks, int s_stride, int mode, uint32_t* status) {
  // One CTA: 32 consecutive rows of every head.  Sixteen lanes read one 16-byte piece each of a row (rows of one
  // head are adjacent in a block, so consecutive lane groups read consecutive memory); the norms pass through
  // shared memory so that the scores are written 32 consecutive floats at a time.  Hkv <= 32 (checked on the host).
  __shared__ float sn[KN_ROWS][33];
  const int seq = blockIdx.z, layer = blockIdx.y;
  const int len = kv_lens[seq];
  const int tok0 = blockIdx.x * KN_ROWS;
  if (tok0 >= len) return;
  const int sub = threadIdx.x & 15, grp = threadIdx.x >> 4;
  const long long kbase = ((long long)layer * 2 + 0) * num_blocks;
  const int* bt = block_tables + (long long)seq * max_blocks;
  const int rows = KN_ROWS * Hkv;
#pragma unroll 4
  for (int r = grp; r < rows; r += 16) {
    const int h = r / KN_ROWS, tl = r % KN_ROWS;
    const int tok = tok0 + tl;
    float ss = 0.f;
    if (tok < len) {
      const int blk = bt[tok / block_size];
      if (blk < 0 || blk >= num_blocks) {
        report(status, ST_BAD_INDEX);
      } else {
        const uint4* row = reinterpret_cast<const uint4*>(
            pool + (((kbase + blk) * Hkv + h) * block_size + tok % block_size) * D);
        for (int i = sub; i < D / 8; i += 16) {
          const uint4 v = row[i];
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {        // a bf16 is the upper half of the fp32 with the same value
            const float a = __uint_as_float(w[e] << 16), b = __uint_as_float(w[e] & 0xffff0000u);
            ss += a * a + b * b;
          }
        }
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (sub == 0) sn[tl][h] = sqrtf(ss);
  }
  __syncthreads();
  float* out = scores + (((long long)seq * L + layer) * Hkv) * s_stride;
  for (int idx = threadIdx.x; idx < rows; idx += 256) {
    const int h = idx / KN_ROWS, tl = idx % KN_ROWS;
    const int tok = tok0 + tl;
    if (tok >= len) continue;
    float v;
    if (mode == 0) {
      v = -sn[tl][h];
    } else {
      float m = 0.f;
      for (int hh = 0; hh < Hkv; ++hh) m += sn[tl][hh];
      v = m / float(Hkv);
    }
    out[(long long)h * s_stride + tok] = v;
  }
}

constexpr int SC_THREADS = 256;
constexpr int SC_CHUNK = 128;

template <int D>
__global__ void __launch_bounds__(SC_THREADS)
select_compact_kernel(bf16* __restrict__ pool, const float* __restrict__ scores,
                      const int* __restrict__ block_tables, const int* __restrict__ kv_lens,
                      const int* __restrict__ n_kepts, int L, int num_blocks, int block_size, int Hkv,
                      int max_blocks, int s_stride, uint32_t* status) {
  extern __shared__ uint32_t sm[];
  const int h = blockIdx.x, layer = blockIdx.y, seq = blockIdx.z;
  const int S = kv_lens[seq];
  int k = n_kepts[seq];
  if (k >= S || S <= 0) return;
  if (k < 1) k = 1;
  uint32_t* keys = sm;                       // [S]
  uint32_t* hist = sm + s_stride;            // [256]
  int* s_misc = reinterpret_cast<int*>(hist + 256);   // [8]: bin, above, ...
  int* wsum = s_misc + 8;                    // [SC_THREADS / 32] warp partials
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const float* sc = scores + (((long long)seq * L + layer) * Hkv + h) * s_stride;
  for (int i = tid; i < S; i += SC_THREADS) keys[i] = float_key(sc[i]);
  __syncthreads();

  // ---- radix select: the k-th largest key
  uint32_t prefix = 0, mask = 0;
  int remaining = k;                         // rank still to find inside the current prefix class
  for (int shift = 24; shift >= 0; shift -= 8) {
    hist[tid] = 0;
    __syncthreads();
    // scores of one request share their leading bits, so most keys of a warp fall into the same bin: the lanes
    // with equal bins elect one that adds their count (one shared-memory atomic per distinct bin and warp)
    for (int i0 = 0; i0 < S; i0 += SC_THREADS) {
      const int i = i0 + tid;
      int bin = -1;
      if (i < S) {
        const uint32_t key = keys[i];
        if ((key & mask) == prefix) bin = int((key >> shift) & 0xFF);
      }
      const unsigned peers = __match_any_sync(0xffffffffu, bin);
      if (bin >= 0 && lane == __ffs(peers) - 1) atomicAdd(&hist[bin], unsigned(__popc(peers)));
    }
    __syncthreads();
    if (warp == 0) {
      // lane l owns bins 255 - 8 l ... 248 - 8 l (from the top); the lane whose bins contain rank `remaining`
      // walks its eight bins
      int mine = 0;
#pragma unroll
      for (int b = 0; b < 8; ++b) mine += int(hist[255 - 8 * lane - b]);
      int x = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      const int above = x - mine;                       // keys in higher bins than this lane's
      const bool here = above < remaining && remaining <= x;
      const unsigned found = __ballot_sync(0xffffffffu, here);
      if (found == 0) {
        if (lane == 31) {                               // fewer keys than `remaining` in this class: lowest bin
          s_misc[0] = 0;
          s_misc[1] = x - int(hist[0]);
        }
      } else if (here) {
        int acc = above, bin = 255 - 8 * lane;
        for (int b = 0; b < 7; ++b, --bin) {
          if (acc + int(hist[bin]) >= remaining) break;
          acc += int(hist[bin]);
        }
        s_misc[0] = bin;
        s_misc[1] = acc;
      }
    }
    __syncthreads();
    prefix |= uint32_t(s_misc[0]) << shift;
    mask |= 0xFFu << shift;
    remaining -= s_misc[1];
    __syncthreads();
  }
  const uint32_t thr = prefix;               // keep key > thr, plus the last `remaining` rows with key == thr
  const int need_eq = remaining;

  // total number of ties
  int eq_local = 0;
  for (int i = tid; i < S; i += SC_THREADS) eq_local += (keys[i] == thr);
  eq_local = int(warp_sum(float(eq_local)) + 0.5f);
  if (lane == 0) wsum[warp] = eq_local;
  __syncthreads();
  int eq_total = 0;
  for (int w = 0; w < SC_THREADS / 32; ++w) eq_total += wsum[w];
  __syncthreads();

  const long long kbase = ((long long)layer * 2 + 0) * num_blocks;
  const long long vbase = ((long long)layer * 2 + 1) * num_blocks;
  const int* bt = block_tables + (long long)seq * max_blocks;
  auto row_ptr = [&](long long base, int tok) -> bf16* {
    const int blk = bt[tok / block_size];
    if (blk < 0 || blk >= num_blocks) {
      report(status, ST_BAD_INDEX);
      return nullptr;
    }
    return pool + (((base + blk) * Hkv + h) * block_size + tok % block_size) * D;
  };

  // ---- destination of every row, once for the whole request: thread t owns rows [t * RPT, (t + 1) * RPT).
  // Two block-wide exclusive scans (ties, then kept rows); afterwards the copy loop needs one barrier per chunk.
  int* dstpos = reinterpret_cast<int*>(keys);            // the keys are no longer needed once a row's flags are known
  const int RPT = (S + SC_THREADS - 1) / SC_THREADS;
  const int r_lo = min(S, tid * RPT), r_hi = min(S, r_lo + RPT);
  auto block_exclusive = [&](int local) -> int {         // exclusive prefix of `local` over the threads of the CTA
    int x = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) wsum[warp] = x;
    __syncthreads();
    int before = x - local;
    for (int w = 0; w < warp; ++w) before += wsum[w];
    __syncthreads();
    return before;
  };
  int eq_mine = 0;
  for (int r = r_lo; r < r_hi; ++r) eq_mine += (keys[r] == thr);
  int eq_before = block_exclusive(eq_mine);
  // a tie is kept when it is among the last `need_eq` ties of the request
  int kept_mine = 0;
  {
    int e = eq_before;
    for (int r = r_lo; r < r_hi; ++r) {
      const uint32_t key = keys[r];
      const bool tie = key == thr;
      kept_mine += (key > thr) || (tie && (eq_total - e) <= need_eq);
      e += tie;
    }
  }
  int pos = block_exclusive(kept_mine);
  {
    int e = eq_before;
    for (int r = r_lo; r < r_hi; ++r) {
      const uint32_t key = keys[r];
      const bool tie = key == thr;
      const bool keep = (key > thr) || (tie && (eq_total - e) <= need_eq);
      e += tie;
      dstpos[r] = keep ? pos : -1;                        // (row r's key is not read again)
      pos += keep;
    }
  }
  __syncthreads();

  // ---- move rows, 128 at a time: read the whole chunk, barrier, write it.  A row only ever moves towards the
  // front, so the rows a chunk writes lie before the rows any LATER chunk reads: no barrier is needed between the
  // writes of one chunk and the reads of the next.
  constexpr int PIECES = D / 8;              // 16-byte pieces per row (K or V)
  constexpr int PER_THREAD = (SC_CHUNK * 2 * PIECES) / SC_THREADS;
  for (int c0 = 0; c0 < S; c0 += SC_CHUNK) {
    uint4 regs[PER_THREAD];
#pragma unroll
    for (int j = 0; j < PER_THREAD; ++j) {
      const int piece = tid + j * SC_THREADS;
      const int r = c0 + piece / (2 * PIECES), part = piece % (2 * PIECES);
      regs[j] = make_uint4(0, 0, 0, 0);
      if (r < S && dstpos[r] >= 0 && dstpos[r] != r) {
        const bf16* src = row_ptr(part < PIECES ? kbase : vbase, r);
        if (src != nullptr) regs[j] = reinterpret_cast<const uint4*>(src)[part % PIECES];
      }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < PER_THREAD; ++j) {
      const int piece = tid + j * SC_THREADS;
      const int r = c0 + piece / (2 * PIECES), part = piece % (2 * PIECES);
      if (r < S && dstpos[r] >= 0 && dstpos[r] != r) {
        bf16* dst = row_ptr(part < PIECES ? kbase : vbase, dstpos[r]);
        if (dst != nullptr) reinterpret_cast<uint4*>(dst)[part % PIECES] = regs[j];
      }
    }
  }
}

void launch_knorm_scores(const void* pool, const int* block_tables, const int* kv_lens, float* scores, int n_seq,
                         int L, int num_blocks, int block_size, int Hkv, int D, int max_blocks, int max_len,
                         int s_stride, int mode, uint32_t* status, cudaStream_t stream) {
  if (n_seq == 0 || max_len == 0) return;
  if (Hkv > 32 || D % 8 != 0) throw std::runtime_error("knorm scores: at most 32 KV heads, head_dim a multiple of 8");
  dim3 grid((max_len + KN_ROWS - 1) / KN_ROWS, L, n_seq);
  knorm_score_kernel<<<grid, 256, 0, stream>>>((const bf16*)pool, block_tables, kv_lens, scores, L, num_blocks,
                                               block_size, Hkv, D, max_blocks, s_stride, mode, status);
}

void launch_select_compact(void* pool, const float* scores, const int* block_tables, const int* kv_lens,
                           const int* n_kepts, int n_seq, int L, int num_blocks, int block_size, int Hkv, int D,
                           int max_blocks, int s_stride, uint32_t* status, cudaStream_t stream) {
  if (n_seq == 0) return;
  dim3 grid(Hkv, L, n_seq);
  const int smem = (s_stride + 256 + 8 + SC_CHUNK + 16) * 4;
  if (smem > 220 * 1024) throw std::runtime_error("select_compact: request too long for one CTA's shared memory");
  auto launch = [&](auto kern) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    kern<<<grid, SC_THREADS, smem, stream>>>((bf16*)pool, scores, block_tables, kv_lens, n_kepts, L, num_blocks,
                                             block_size, Hkv, max_blocks, s_stride, status);
  };
  if (D == 128) launch(select_compact_kernel<128>);
  else if (D == 64) launch(select_compact_kernel<64>);
  else throw std::runtime_error("select_compact: head_dim must be 64 or 128");
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("select_compact launch: ") + cudaGetErrorString(e));
}

}  // namespace fc
