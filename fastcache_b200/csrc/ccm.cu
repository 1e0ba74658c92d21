// Fused CCM merge compressor operating in the paged KV pool (head_dim 128).
//
// For one (request, group of G kv heads, layer, K|V) a CTA walks the request's rows in
// ascending order, segment by segment (image rows first, then text rows, each with its own
// MLP bank): f consecutive rows of a head are concatenated (they are adjacent in the
// head-major pool, so the "concatenation" is only an addressing rule), pushed through
//        y = W3 relu(W2 relu(W1 z + b1) + b2) + b3
// and written to the leading rows of the same request; the (rows mod f) remainder of a
// segment is moved unchanged.  A tile is 128 output rows: 128 / G consecutive output rows of
// each of the G heads (the MLP weights are shared by all heads, so short segments still fill
// the 128-row tensor-core tile; the host picks G from the segment lengths).
//
//   warps 2-5 (128 workers)  gather the A operand k-block by k-block with cp.async into the
//                            128-byte-swizzled layout tcgen05 expects (up to three k-blocks
//                            in flight), run the epilogues (tcgen05.ld, bias, ReLU, bf16) and
//                            scatter the result rows
//   warp 0                   streams W1 / W2 / W3 k-blocks with TMA into the same stage ring
//   warp 1                   issues tcgen05.mma: GEMM1 over f*2 k-blocks (A gathered), GEMM2 and
//                            GEMM3 with the activation tile as the A operand; the epilogue writes
//                            that tile into the A halves of the two stages whose W halves carry
//                            the matching W2 / W3 k-blocks (those halves are idle then), so the
//                            CTA needs 96 KiB and two CTAs share an SM; accumulators live in TMEM
// The intermediates never leave the SM.  In-place safety: an output row index never
// exceeds the index of any input row of the same head it depends on, tiles are processed in
// ascending order by one CTA, and a tile is read completely (GEMM1 is done) before it is written.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

#include "gemm.h"
#include "kernels.h"
#include "mma.cuh"
#include "ptx.cuh"

namespace fc {

using bf16 = __nv_bfloat16;

constexpr int CCM_D = 128;
constexpr int CCM_STAGES = 3;
constexpr int CCM_THREADS = 192;
constexpr int CCM_TILE = 128;          // output rows per tile
constexpr int CCM_KB_BYTES = CCM_TILE * 64 * 2;   // one [128 x 64] bf16 sub-tile

struct CcmParams {
  bf16* pool;                 // [L, 2, num_blocks, Hkv, block_size, D]
  const int* block_tables;    // [n_seq, max_blocks]
  const int* dst_tables;      // [n_seq, max_blocks] blocks the result is written to, or nullptr: in place
  const int* kv_lens;         // [n_seq]
  const int* image_lens;      // [n_seq]
  const bf16 *b1, *b2, *b3;   // [Lw, 4, D]
  int num_blocks, Hkv, block_size, max_blocks;
  int layer_start;            // first pool layer handled by blockIdx.y / 2 == 0
  int weight_layer_start;     // index of that layer in the packed weights
  int factor, min_seq_len;
  int single_segment;
  int heads_per_cta;          // G: 1, 2, 4 or 8 heads share a tile
  int rj_shift;               // log2(128 / G): output rows of one head per tile
  uint32_t* status;
};

__device__ __forceinline__ int ccm_seg_out(int n, int f, int min_len) {
  if (n <= 0) return 0;
  const int s = n / f;
  return s < min_len ? n : s + n % f;
}

__global__ void __launch_bounds__(CCM_THREADS, 2)
ccm_fused_kernel(const __grid_constant__ CUtensorMap tm_w1, const __grid_constant__ CUtensorMap tm_w2,
                 const __grid_constant__ CUtensorMap tm_w3, const CcmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // stage s: A sub-tile at s * 2 * KB, W sub-tile right after
  uint64_t* a_full = reinterpret_cast<uint64_t*>(smem + CCM_STAGES * 2 * CCM_KB_BYTES);
  uint64_t* w_full = a_full + CCM_STAGES;
  uint64_t* empty = w_full + CCM_STAGES;
  uint64_t* acc_full = empty + CCM_STAGES;      // [1]
  uint64_t* h_ready = acc_full + 1;             // [1]
  uint64_t* acc_free = h_ready + 1;             // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 1);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.heads_per_cta, rj_shift = p.rj_shift, RJ = 1 << rj_shift;
  const int h0 = blockIdx.x * G, seq = blockIdx.z;
  const int layer_off = blockIdx.y >> 1, kv = blockIdx.y & 1;
  const int layer = p.layer_start + layer_off, wlayer = p.weight_layer_start + layer_off;
  const int f = p.factor;
  const int nk1 = f * (CCM_D / 64);             // k-blocks of GEMM1
  const int nk_tile = nk1 + 4;                  // + 2 for W2 + 2 for W3

  if (threadIdx.x == 0) {
    for (int s = 0; s < CCM_STAGES; ++s) {
      mbar_init(&a_full[s], 128);
      mbar_init(&w_full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(h_ready, 128);
    mbar_init(acc_free, 128);
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_w1);
    tma_prefetch_desc(&tm_w2);
    tma_prefetch_desc(&tm_w3);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // ---- the request's segments (identical arithmetic in every role)
  const int S = p.kv_lens[seq];
  int img = p.single_segment ? 0 : p.image_lens[seq];
  img = max(0, min(img, S));
  const int seg_in[2] = {0, img};
  const int seg_len[2] = {img, S - img};
  const int seg_out[2] = {0, ccm_seg_out(img, f, p.min_seq_len)};
  int seg_tiles[2];
  for (int s = 0; s < 2; ++s) {
    const int sp = seg_len[s] / f;
    seg_tiles[s] = (seg_len[s] > 0 && sp >= p.min_seq_len) ? (sp + RJ - 1) >> rj_shift : 0;
  }
  const int total_tiles = seg_tiles[0] + seg_tiles[1];

  const int* bt = p.block_tables + (long long)seq * p.max_blocks;
  const long long plane = (((long long)layer * 2 + kv) * p.num_blocks);
  auto row_ptr = [&](int hh, int tok) -> bf16* {
    int blk = bt[tok / p.block_size];
    if (blk < 0 || blk >= p.num_blocks) {
      report(p.status, ST_BAD_INDEX);
      return nullptr;
    }
    return p.pool + (((plane + blk) * p.Hkv + hh) * p.block_size + tok % p.block_size) * CCM_D;
  };
  // destination rows: the request's own blocks (in place), or a second set of blocks, in which case the
  // source rows stay intact and the request can keep decoding over them while its layers are compressed
  const bool out_of_place = p.dst_tables != nullptr;
  const int* dbt = out_of_place ? p.dst_tables + (long long)seq * p.max_blocks : bt;
  auto dst_ptr = [&](int hh, int tok) -> bf16* {
    int blk = dbt[tok / p.block_size];
    if (blk < 0 || blk >= p.num_blocks) {
      report(p.status, ST_BAD_INDEX);
      return nullptr;
    }
    return p.pool + (((plane + blk) * p.Hkv + hh) * p.block_size + tok % p.block_size) * CCM_D;
  };

  if (warp == 0) {
    // ------------------------------------------------------------- weight producer (TMA)
    if (lane == 0) {
      int it = 0;
      for (int tile = 0; tile < total_tiles && !*s_abort; ++tile) {
        const int seg = tile < seg_tiles[0] ? 0 : 1;
        const int bank = (seg == 0 ? 2 : 0) + kv;             // (tk, tv, ik, iv)
        const int wrow = (wlayer * 4 + bank) * CCM_D;
        for (int i = 0; i < nk_tile; ++i, ++it) {
          const int stage = it % CCM_STAGES;
          if (!mbar_wait(&empty[stage], ((it / CCM_STAGES) & 1) ^ 1, p.status, ST_TIMEOUT_EMPTY)) {
            *s_abort = 1;
            break;
          }
          uint8_t* sw = smem + stage * 2 * CCM_KB_BYTES + CCM_KB_BYTES;
          mbar_expect_tx(&w_full[stage], CCM_KB_BYTES);
          if (i < nk1) tma_load_2d(sw, &tm_w1, &w_full[stage], i * 64, wrow);
          else if (i < nk1 + 2) tma_load_2d(sw, &tm_w2, &w_full[stage], (i - nk1) * 64, wrow);
          else tma_load_2d(sw, &tm_w3, &w_full[stage], (i - nk1 - 2) * 64, wrow);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, 128);
      int it = 0;
      uint32_t h_phase = 0, free_phase = 0;
      uint32_t a_uses[CCM_STAGES] = {0, 0, 0};
      bool ok = true;
      for (int tile = 0; tile < total_tiles && ok; ++tile) {
        // the previous tile's last epilogue must have drained accumulator 0
        if (tile > 0) {
          ok = mbar_wait(acc_free, free_phase, p.status, ST_TIMEOUT_ACC_EMPTY);
          free_phase ^= 1;
          if (!ok) break;
          tc_fence_after();
        }
        for (int g = 0; g < 3 && ok; ++g) {
          const int nk = g == 0 ? nk1 : 2;
          const uint32_t d_tmem = tmem_base + (g == 1 ? 128u : 0u);
          if (g > 0) {
            ok = mbar_wait(h_ready, h_phase, p.status, ST_TIMEOUT_ACC_FULL);
            h_phase ^= 1;
            if (!ok) break;
            tc_fence_after();
          }
          for (int i = 0; i < nk && ok; ++i, ++it) {
            const int stage = it % CCM_STAGES;
            const uint32_t ph = (it / CCM_STAGES) & 1;
            ok = mbar_wait(&w_full[stage], ph, p.status, ST_TIMEOUT_FULL);
            if (ok && g == 0) {
              // a_full[stage] completes a phase only when the stage carries a gathered operand,
              // so its parity is counted per stage, not derived from the ring position
              ok = mbar_wait(&a_full[stage], a_uses[stage] & 1u, p.status, ST_TIMEOUT_FULL);
              ++a_uses[stage];
            }
            if (!ok) break;
            tc_fence_after();
            // the A half of the stage holds the gathered rows (GEMM1) or the activation sub-tile that the
            // epilogue wrote for this k-block (GEMM2, GEMM3)
            const uint32_t sa = smem_u32(smem + stage * 2 * CCM_KB_BYTES);
            const uint64_t da = make_sdesc_sw128(sa);
            const uint64_t db = make_sdesc_sw128(sa + CCM_KB_BYTES);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              tc_mma_f16(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), idesc, (i > 0 || k > 0) ? 1u : 0u);
            tc_commit(&empty[stage]);
          }
          if (ok) tc_commit(acc_full);
        }
      }
      if (!ok) *s_abort = 1;
    }
  } else {
    // --------------------------------------------------- workers: gather, epilogues, scatter
    const int wt = threadIdx.x - 64;               // 0..127
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;        // TMEM lane == tile row owned by this thread
    int it = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    int tile = 0;
    for (int seg = 0; seg < 2 && ok; ++seg) {
      const int n = seg_len[seg];
      if (n <= 0) continue;
      const int sp = n / f;
      const int in0 = seg_in[seg], out0 = seg_out[seg];
      if (seg_tiles[seg] == 0) {
        // too short to compress: move the rows unchanged (at most a few rows; out0 <= in0)
        if (out0 != in0 || out_of_place) {
          for (int hl = 0; hl < G; ++hl) {
            for (int base = 0; base < n; base += 8) {
              const int r = base + wt / 16, piece = wt % 16;
              uint4 v = make_uint4(0, 0, 0, 0);
              const bool live = r < n;
              if (live) {
                const bf16* src = row_ptr(h0 + hl, in0 + r);
                if (src != nullptr) v = reinterpret_cast<const uint4*>(src)[piece];
              }
              asm volatile("bar.sync 1, 128;" ::: "memory");
              if (live) {
                bf16* dst = dst_ptr(h0 + hl, out0 + r);
                if (dst != nullptr) reinterpret_cast<uint4*>(dst)[piece] = v;
              }
              asm volatile("bar.sync 1, 128;" ::: "memory");
            }
          }
        }
        continue;
      }
      const int bank = (seg == 0 ? 2 : 0) + kv;
      const bf16* b1 = p.b1 + ((long long)wlayer * 4 + bank) * CCM_D;
      const bf16* b2 = p.b2 + ((long long)wlayer * 4 + bank) * CCM_D;
      const bf16* b3 = p.b3 + ((long long)wlayer * 4 + bank) * CCM_D;
      for (int t = 0; t < seg_tiles[seg] && ok; ++t, ++tile) {
        const int j0 = t << rj_shift;
        // ---- gather the A operand of GEMM1, one [128 x 64] k-block per stage; the copies of up to three
        //      k-blocks are in flight, a stage is handed to the MMA warp when its own group has landed
        for (int i = 0; i < nk1 && ok; ++i, ++it) {
          const int stage = it % CCM_STAGES;
          if (*s_abort || !mbar_wait(&empty[stage], ((it / CCM_STAGES) & 1) ^ 1, p.status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_u32(smem + stage * 2 * CCM_KB_BYTES);
          const int tok_in_group = i / (CCM_D / 64), half = i % (CCM_D / 64);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int c = wt + q * 128;              // 1024 chunks of 16 bytes: (tile row r, chunk ch)
            const int r = c >> 3, ch = c & 7;
            const int j = j0 + (r & (RJ - 1));       // tile row r = head (r >> rj_shift), output row j of that head
            const bf16* src = p.pool;
            bool live = j < sp;
            if (live) {
              const bf16* rp = row_ptr(h0 + (r >> rj_shift), in0 + j * f + tok_in_group);
              if (rp == nullptr) live = false;
              else src = rp + half * 64 + ch * 8;
            }
            cp_async16(sa + r * 128 + ((ch ^ (r & 7)) << 4), src, live);
          }
          cp_async_commit();
          if (i >= 2) {
            cp_async_wait<2>();
            fence_proxy_async();
            mbar_arrive(&a_full[(it - 2) % CCM_STAGES]);
          }
        }
        cp_async_wait<0>();
        if (!ok) break;
        // the last two k-blocks (GEMM1 always has at least two)
        fence_proxy_async();
        mbar_arrive(&a_full[(it - 2) % CCM_STAGES]);
        mbar_arrive(&a_full[(it - 1) % CCM_STAGES]);
        const int it_h = it;     // ring position of the first W2 k-block: its stage takes the first activation sub-tile
        it += 4;     // the W2 / W3 stages carry no gathered operand (the MMA warp counts a_full uses per stage)
        // ---- epilogues 1 and 2: bias + ReLU, activation tile to shared memory for the next GEMM
        for (int g = 0; g < 2 && ok; ++g) {
          if (!mbar_wait(acc_full, acc_phase, p.status, ST_TIMEOUT_ACC_FULL)) {
            ok = false;
            break;
          }
          acc_phase ^= 1;
          tc_fence_after();
          const bf16* bias = g == 0 ? b1 : b2;
          const uint32_t t_addr = tmem_base + (uint32_t(lane_group * 32) << 16) + (g == 1 ? 128u : 0u);
          // activation sub-tile i (columns 64 i .. 64 i + 63) goes to the A half of the stage whose W half
          // carries k-block i of the next GEMM; every earlier use of those halves is complete (acc_full)
          uint8_t* const h_dst0 = smem + ((it_h + 2 * g) % CCM_STAGES) * 2 * CCM_KB_BYTES;
          uint8_t* const h_dst1 = smem + ((it_h + 2 * g + 1) % CCM_STAGES) * 2 * CCM_KB_BYTES;
#pragma unroll 1
          for (int c4 = 0; c4 < 4; ++c4) {
            uint32_t rr[32];
            tmem_ld_32x32(t_addr + uint32_t(c4 * 32), rr);
            tmem_ld_wait();
            uint8_t* const h_row = (c4 < 2 ? h_dst0 : h_dst1) + row * 128;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 bv = *reinterpret_cast<const uint4*>(bias + c4 * 32 + q * 8);
              const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
              uint32_t u[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                // a bf16 is the upper half of the fp32 with the same value
                const float a = fmaxf(__uint_as_float(rr[q * 8 + e * 2]) + __uint_as_float(bw[e] << 16), 0.f);
                const float b = fmaxf(__uint_as_float(rr[q * 8 + e * 2 + 1]) + __uint_as_float(bw[e] & 0xffff0000u), 0.f);
                u[e] = pack_bf16(a, b);
              }
              const int chunk = (c4 & 1) * 4 + q;      // 16-byte chunk of the 128-byte sub-tile row
              *reinterpret_cast<uint4*>(h_row + ((chunk ^ (row & 7)) << 4)) = make_uint4(u[0], u[1], u[2], u[3]);
            }
          }
          tc_fence_before();
          fence_proxy_async();
          mbar_arrive(h_ready);
        }
        if (!ok) break;
        // ---- epilogue 3: bias, bf16, scatter the rows of this tile
        if (!mbar_wait(acc_full, acc_phase, p.status, ST_TIMEOUT_ACC_FULL)) {
          ok = false;
          break;
        }
        acc_phase ^= 1;
        tc_fence_after();
        {
          const int j = j0 + (row & (RJ - 1));
          bf16* dst = (j < sp) ? dst_ptr(h0 + (row >> rj_shift), out0 + j) : nullptr;
          const uint32_t t_addr = tmem_base + (uint32_t(lane_group * 32) << 16);
#pragma unroll 1
          for (int c4 = 0; c4 < 4; ++c4) {
            uint32_t rr[32];
            tmem_ld_32x32(t_addr + uint32_t(c4 * 32), rr);
            tmem_ld_wait();
            if (dst != nullptr) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 bv = *reinterpret_cast<const uint4*>(b3 + c4 * 32 + q * 8);
                const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
                uint32_t u[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  u[e] = pack_bf16(__uint_as_float(rr[q * 8 + e * 2]) + __uint_as_float(bw[e] << 16),
                                   __uint_as_float(rr[q * 8 + e * 2 + 1]) + __uint_as_float(bw[e] & 0xffff0000u));
                }
                reinterpret_cast<uint4*>(dst)[c4 * 4 + q] = make_uint4(u[0], u[1], u[2], u[3]);
              }
            }
          }
        }
        tc_fence_before();
        mbar_arrive(acc_free);
      }
      if (!ok) break;
      // ---- remainder rows of the segment move behind the compressed rows (fewer than f rows)
      const int rem = n - sp * f;
      if (rem > 0) {
        for (int hl = 0; hl < G; ++hl) {
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const int r = wt / 16, piece = wt % 16;
          uint4 v = make_uint4(0, 0, 0, 0);
          const bool live = r < rem;
          if (live) {
            const bf16* src = row_ptr(h0 + hl, in0 + sp * f + r);
            if (src != nullptr) v = reinterpret_cast<const uint4*>(src)[piece];
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (live) {
            bf16* dst = dst_ptr(h0 + hl, out0 + sp + r);
            if (dst != nullptr) reinterpret_cast<uint4*>(dst)[piece] = v;
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      __threadfence_block();
    }
    if (!ok) *s_abort = 1;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// Weights: w1 [Lw, 4, D, D*f], w2 / w3 [Lw, 4, D, D], biases [Lw, 4, D]; bf16, contiguous.
void launch_ccm_fused(void* pool, const int* block_tables, const int* kv_lens, const int* image_lens,
                      const void* w1, const void* w2, const void* w3, const void* b1, const void* b2,
                      const void* b3, int n_seq, int n_weight_layers, int layer_start, int layer_end,
                      int weight_layer_start, int num_blocks, int Hkv, int block_size, int D, int max_blocks,
                      int factor, int min_seq_len, int single_segment, int heads_per_cta, uint32_t* status,
                      cudaStream_t stream, const int* dst_block_tables) {
  if (n_seq == 0 || layer_end <= layer_start) return;
  int G = heads_per_cta <= 0 ? 1 : heads_per_cta;
  if ((G != 1 && G != 2 && G != 4 && G != 8) || Hkv % G != 0)
    throw std::runtime_error("fused CCM kernel: heads per CTA must be 1, 2, 4 or 8 and divide the KV heads");
  int rj_shift = 7;
  for (int g = G; g > 1; g >>= 1) --rj_shift;
  if (D != CCM_D) throw std::runtime_error("fused CCM kernel: head_dim must be 128");
  if (factor < 1 || factor > 8) throw std::runtime_error("fused CCM kernel: factor must be in [1, 8]");
  if (factor > 8) throw std::runtime_error("remainder move handles fewer than 8 rows");
  CcmParams p{};
  p.pool = (bf16*)pool;
  p.block_tables = block_tables;
  p.dst_tables = dst_block_tables;
  p.kv_lens = kv_lens;
  p.image_lens = image_lens;
  p.b1 = (const bf16*)b1;
  p.b2 = (const bf16*)b2;
  p.b3 = (const bf16*)b3;
  p.num_blocks = num_blocks;
  p.Hkv = Hkv;
  p.block_size = block_size;
  p.max_blocks = max_blocks;
  p.layer_start = layer_start;
  p.weight_layer_start = weight_layer_start;
  p.factor = factor;
  p.min_seq_len = min_seq_len;
  p.single_segment = single_segment;
  p.heads_per_cta = G;
  p.rj_shift = rj_shift;
  p.status = status;
  const uint64_t wrows = (uint64_t)n_weight_layers * 4 * D;
  const CUtensorMap t1 = make_tmap_bf16_2d(w1, wrows, (uint64_t)D * factor, (uint64_t)D * factor, 128, 64);
  const CUtensorMap t2 = make_tmap_bf16_2d(w2, wrows, D, D, 128, 64);
  const CUtensorMap t3 = make_tmap_bf16_2d(w3, wrows, D, D, 128, 64);
  const int smem = CCM_STAGES * 2 * CCM_KB_BYTES + 256 + 1024;
  cudaFuncSetAttribute(ccm_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  dim3 grid(Hkv / G, (layer_end - layer_start) * 2, n_seq);
  ccm_fused_kernel<<<grid, CCM_THREADS, smem, stream>>>(t1, t2, t3, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("fused CCM launch: ") + cudaGetErrorString(e));
}

}  // namespace fc
