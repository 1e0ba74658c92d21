// Dense (non-causal) attention on tcgen05 for the vision towers and the resampler: head_dim up to 128.
//
// out[b, s, h, :] = softmax(q[b, s, h, :] . k[b, :, h, :]^T * scale  (+ key mask)) v[b, :, h, :]
//
// Same structure as the causal prefill kernel (attn_prefill_tc2.cu): one CTA owns 256 query rows of one head
// of one batch element (tiles A and B of 128 rows, in ping-pong) and walks the keys in tiles of 128 rows; S, P
// and O live in tensor memory:
//     S_A [0,128)  S_B [128,256)  O_A [256,256+DP)  O_B [256+DP,256+2DP)
//   warp 0       TMA: both Q tiles once, then K and V tiles into 2-stage rings (128-byte swizzle)
//   warp 1       tcgen05.mma issuer: S_X = Q_X K^T from shared memory, O_X += P_X V with P_X read from tensor
//                memory (packed bf16 over the first 64 columns of S_X) and V as an MN-major operand
//   warps 2-5    softmax of tile A, warps 6-9 of tile B, one query row per thread, O rescaled lazily
//
// The operands are [B, S, H, D] views with arbitrary strides (the packed qkv output of one GEMM is read in place),
// described to TMA as 4-D tensors (D, H, S, B).  The head dimension is padded to DP = 64 or 128 columns by the
// copy itself: elements past D, and rows past S, are outside the tensor and arrive as zeros, so head_dim 72
// (SigLIP) runs as 128 with zero columns that add nothing to S and produce O columns that are not written.
// The box starts at x = 0 or 64 elements, i.e. on 16-byte boundaries.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>
#include <stdexcept>
#include <string>

#include "gemm.h"
#include "kernels.h"
#include "ptx.cuh"

namespace fc {

using bf16 = __nv_bfloat16;

constexpr int DT_BM = 128;             // rows per query tile (two tiles per CTA)
constexpr int DT_BN = 128;
constexpr int DT_THREADS = 320;
constexpr int DT_THREADS_SINGLE = 192;
constexpr int DT_SUB_BYTES = 128 * 64 * 2;              // one [128 x 64] sub-tile
constexpr float DT_RESCALE_THRESHOLD = 8.f;             // log2 units

__device__ __forceinline__ uint64_t dt_sdesc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((addr & 0x3FFFF) >> 4);
  d |= uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}

__device__ __forceinline__ float dt_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ void dt_tma_load_4d(void* smem, const CUtensorMap* m, uint64_t* bar, int x, int y, int z,
                                               int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

struct DenseTcParams {
  bf16* out;                 // [B, Sq, H, D] contiguous
  const uint8_t* key_mask;   // [B, mask_ld] (1 = attend), rows padded with zeros to a multiple of 128; or null
  int mask_ld;
  int Sq, Sk, H, D;
  float scale_log2;
  uint32_t* status;
};

// PAIR: two query tiles per CTA in ping-pong, one CTA per SM (512 columns of tensor memory).  Otherwise one query
// tile per CTA, half the tensor memory and (for DP = 64) half the shared memory, so that two CTAs share an SM:
// the start-up and the epilogue of one overlap the key loop of the other, and a sequence of 577 rows costs five
// tiles instead of three pairs.
template <int DP, bool PAIR>
__global__ void __launch_bounds__(PAIR ? DT_THREADS : DT_THREADS_SINGLE, PAIR ? 1 : 2)
dense_attn_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const DenseTcParams p) {
  constexpr int SUBS = DP / 64;
  constexpr int TILE_BYTES = SUBS * DT_SUB_BYTES;
  constexpr int NQ = PAIR ? 2 : 1;                     // query tiles per CTA
  constexpr uint32_t O_BASE = PAIR ? 256u : 128u;      // first column of O_A
  constexpr uint32_t TMEM_COLS = PAIR ? 512u : 256u;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem;                                // 2 tiles
  uint8_t* s_k = s_q + NQ * TILE_BYTES;               // 2 stages
  uint8_t* s_v = s_k + 2 * TILE_BYTES;                // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_v + 2 * TILE_BYTES);
  uint64_t* q_full = bars;            // [1]
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [2] per query tile
  uint64_t* p_ready = bars + 11;      // [2] per query tile (128 arrivals)
  uint64_t* o_done = bars + 13;       // [2] per query tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int q0 = blockIdx.x * (NQ * DT_BM);
  const bool act_b = PAIR && q0 + DT_BM < p.Sq;
  const int n_tiles = (p.Sk + DT_BN - 1) / DT_BN;
  const int n_a = n_tiles, n_b = act_b ? n_tiles : 0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_ready[s], 128);
      mbar_init(&o_done[s], 1);
    }
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA loader
    if (lane == 0) {
      mbar_expect_tx(q_full, (act_b ? 2 : 1) * TILE_BYTES);
      for (int x = 0; x < (act_b ? 2 : 1); ++x)
        for (int sub = 0; sub < SUBS; ++sub)
          dt_tma_load_4d(s_q + x * TILE_BYTES + sub * DT_SUB_BYTES, &tm_q, q_full, sub * 64, h, q0 + x * DT_BM, b);
      for (int j = 0; j < n_tiles && !*s_abort; ++j) {
        const int st = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        for (int which = 0; which < 2; ++which) {
          uint64_t* full = which == 0 ? &k_full[st] : &v_full[st];
          uint64_t* empty = which == 0 ? &k_empty[st] : &v_empty[st];
          if (!mbar_wait(empty, ph, p.status, ST_TIMEOUT_EMPTY)) {
            *s_abort = 1;
            break;
          }
          uint8_t* dst = (which == 0 ? s_k : s_v) + st * TILE_BYTES;
          const CUtensorMap* tm = which == 0 ? &tm_k : &tm_v;
          mbar_expect_tx(full, TILE_BYTES);           // rows and columns outside the tensor count as copied zeros
          for (int sub = 0; sub < SUBS; ++sub)
            dt_tma_load_4d(dst + sub * DT_SUB_BYTES, tm, full, sub * 64, h, j * DT_BN, b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, DP, false, true);      // B (= V) is MN-major
      bool ok = mbar_wait(q_full, 0, p.status, ST_TIMEOUT_FULL);
      auto issue_s = [&](int x, int j) {
        const int st = j & 1;
        const uint32_t qa = smem_u32(s_q + x * TILE_BYTES), ka = smem_u32(s_k + st * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk) {
          const uint32_t off = uint32_t(kk >> 2) * DT_SUB_BYTES + uint32_t(kk & 3) * 32;
          tc_mma_f16(tmem_base + uint32_t(x * 128), dt_sdesc(qa + off, 16, 1024), dt_sdesc(ka + off, 16, 1024),
                     idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[x]);
      };
      auto issue_pv = [&](int x, int j) {
        const int st = j & 1;
        const uint32_t va = smem_u32(s_v + st * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t db = dt_sdesc(va + uint32_t(kk) * 2048, DT_SUB_BYTES, 1024);
          tc_mma_f16_ts(tmem_base + O_BASE + uint32_t(x * DP), tmem_base + uint32_t(x * 128) + uint32_t(kk * 8), db,
                        idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&o_done[x]);
      };
      if (ok) ok = mbar_wait(&k_full[0], 0, p.status, ST_TIMEOUT_FULL);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        if (act_b) issue_s(1, 0);
        tc_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        const bool more = j + 1 < n_tiles;
        bool v_waited = false, k_waited = false;
        for (int x = 0; x < 2 && ok; ++x) {
          const int n_x = x == 0 ? n_a : n_b;
          if (j >= n_x) continue;
          ok = mbar_wait(&p_ready[x], uint32_t(j) & 1u, p.status, ST_TIMEOUT_FULL);
          if (ok && !v_waited) {
            ok = mbar_wait(&v_full[st], uint32_t(j >> 1) & 1u, p.status, ST_TIMEOUT_FULL);
            v_waited = true;
          }
          if (!ok) break;
          tc_fence_after();
          issue_pv(x, j);
          if (j + 1 < n_x) {
            if (!k_waited) {
              ok = mbar_wait(&k_full[st ^ 1], uint32_t((j + 1) >> 1) & 1u, p.status, ST_TIMEOUT_FULL);
              k_waited = true;
              if (!ok) break;
              tc_fence_after();
            }
            issue_s(x, j + 1);
          }
        }
        if (!ok) break;
        tc_commit(&v_empty[st]);
        if (more && k_waited) tc_commit(&k_empty[st ^ 1]);
      }
      if (!ok) *s_abort = 1;
    }
  } else {
    // ------------------------------------------------ softmax of one query tile (x = 0: A, 1: B)
    const int x = (warp - 2) >> 2;
    const int n_x = x == 0 ? n_a : n_b;
    const int lane_group = warp & 3;                         // TMEM lanes this warp may touch
    const int row = lane_group * 32 + lane;
    const uint32_t lane_addr = uint32_t(lane_group * 32) << 16;
    const uint32_t ts = tmem_base + lane_addr + uint32_t(x * 128);           // S_x, then P_x
    const uint32_t to = tmem_base + lane_addr + O_BASE + uint32_t(x * DP);   // O_x
    const int qrow = q0 + x * DT_BM + row;
    const uint8_t* mrow = p.key_mask != nullptr ? p.key_mask + (long long)b * p.mask_ld : nullptr;
    float m_ref = 0.f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_x && ok; ++j) {
      if (*s_abort || !mbar_wait(&s_full[x], uint32_t(j) & 1u, p.status, ST_TIMEOUT_ACC_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(ts + uint32_t(c * 32), *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
      tmem_ld_wait();
      const int col0 = j * DT_BN;
      if (mrow != nullptr) {
        // the same 128 bytes for every row of the tile: broadcast loads, served by L1 after the first warp
        const uint4* m4 = reinterpret_cast<const uint4*>(mrow + col0);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const uint4 mv = __ldg(m4 + g);
          const uint32_t w[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
          for (int t = 0; t < 16; ++t)
            if (((w[t >> 2] >> ((t & 3) * 8)) & 0xffu) == 0u) s[g * 16 + t] = 0xff800000u;      // -inf
        }
      } else if (col0 + DT_BN > p.Sk) {
#pragma unroll
        for (int t = 0; t < 128; ++t)
          if (col0 + t >= p.Sk) s[t] = 0xff800000u;
      }
      // four independent chains each (a single one is 128 dependent operations per tile)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int t = 0; t < 128; t += 8) {
#pragma unroll
        for (int i = 0; i < 4; ++i) mx4[i] = dt_max3(mx4[i], __uint_as_float(s[t + 2 * i]), __uint_as_float(s[t + 2 * i + 1]));
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= p.scale_log2;
      if (j == 0) {
        m_ref = (mx == -INFINITY) ? 0.f : mx;
      } else if (__any_sync(__activemask(), mx > m_ref + DT_RESCALE_THRESHOLD)) {
        // some row of this warp outgrew its reference: bring O (complete up to tile j - 1) to the new one
        if (!mbar_wait(&o_done[x], uint32_t(j - 1) & 1u, p.status, ST_TIMEOUT_ACC_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const float m_new = fmaxf(m_ref, mx);
        const float f = exp2f(m_ref - m_new);
        m_ref = m_new;
        l *= f;
#pragma unroll 1
        for (int c = 0; c < DP / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(to + uint32_t(c * 32), r);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 32; ++t) r[t] = __float_as_uint(__uint_as_float(r[t]) * f);
          tmem_st_32x32(to + uint32_t(c * 32), r);
        }
        tmem_st_wait();
      }
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t u[64];
#pragma unroll
      for (int t = 0; t < 64; ++t) {
        float e0, e1;
        const float a0 = fmaf(__uint_as_float(s[2 * t]), p.scale_log2, -m_ref);
        const float a1 = fmaf(__uint_as_float(s[2 * t + 1]), p.scale_log2, -m_ref);
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(a0));
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(a1));
        rs4[t & 3] += e0 + e1;
        u[t] = pack_bf16(e0, e1);
      }
      const float rs = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      tmem_st_32x32(ts, *reinterpret_cast<uint32_t(*)[32]>(&u[0]));
      tmem_st_32x32(ts + 32u, *reinterpret_cast<uint32_t(*)[32]>(&u[32]));
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_ready[x]);
      l += rs;
    }
    if (!ok) *s_abort = 1;
    if (ok && n_x > 0 && mbar_wait(&o_done[x], uint32_t(n_x - 1) & 1u, p.status, ST_TIMEOUT_ACC_FULL)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = p.out + (((long long)b * p.Sq + qrow) * p.H + h) * p.D;
#pragma unroll 1
      for (int c = 0; c < DP / 32; ++c) {
        if (c * 32 >= p.D) break;                       // uniform over the warp
        uint32_t r[32];
        tmem_ld_32x32(to + uint32_t(c * 32), r);
        tmem_ld_wait();
        if (qrow < p.Sq) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (c * 32 + q * 8 < p.D) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(r[q * 8 + 0]) * inv, __uint_as_float(r[q * 8 + 1]) * inv);
              v.y = pack_bf16(__uint_as_float(r[q * 8 + 2]) * inv, __uint_as_float(r[q * 8 + 3]) * inv);
              v.z = pack_bf16(__uint_as_float(r[q * 8 + 4]) * inv, __uint_as_float(r[q * 8 + 5]) * inv);
              v.w = pack_bf16(__uint_as_float(r[q * 8 + 6]) * inv, __uint_as_float(r[q * 8 + 7]) * inv);
              reinterpret_cast<uint4*>(dst + c * 32)[q] = v;
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

// 4-D bf16 view (D, H, S, B) of a [B, S, H, D] tensor with element strides (sb, ss, sh, 1); box = 64 x 1 x 128 x 1
static CUtensorMap dt_tmap(const void* base, int B, int S, int H, int D, const long long* strides) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
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
  CUtensorMap m;
  cuuint64_t dims[4] = {cuuint64_t(D), cuuint64_t(H), cuuint64_t(S), cuuint64_t(B)};
  cuuint64_t str[3] = {cuuint64_t(strides[2]) * 2, cuuint64_t(strides[1]) * 2, cuuint64_t(strides[0]) * 2};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, str, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw std::runtime_error("dense attention: cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
  return m;
}

bool dense_attention_tc_supported(int B, int Sq, int Sk, int H, int D, const long long* q_strides,
                                  const long long* k_strides, const long long* v_strides) {
  if (D % 8 != 0 || D > 128 || D < 8 || Sk < 1 || Sq < 1) return false;
  for (const long long* s : {q_strides, k_strides, v_strides}) {
    // TMA wants strides that are positive multiples of 16 bytes (an expanded view has 0), each a multiple of the
    // one below it; a dimension of extent 1 gets a stride of its own at launch
    const long long sb = s[0], ss = s[1], sh = s[2];
    if (ss <= 0 || ss % 8 != 0) return false;
    if (H > 1 && (sh <= 0 || sh % 8 != 0 || sh < D || ss % sh != 0 || ss < sh * H)) return false;
    if (H == 1 && ss < D) return false;
    if (B > 1 && (sb <= 0 || sb % ss != 0)) return false;
  }
  return true;
}

template <int DP, bool PAIR>
static void dt_launch(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const DenseTcParams& p,
                      dim3 grid, cudaStream_t stream) {
  constexpr int smem = ((PAIR ? 2 : 1) + 4) * (DP / 64) * DT_SUB_BYTES + 256 + 1024;
  auto kern = dense_attn_tc_kernel<DP, PAIR>;
  static std::atomic<uint64_t> configured{0};
  int dev = 0;
  cudaGetDevice(&dev);
  const uint64_t bit = 1ull << (dev & 63);
  if (!(configured.load(std::memory_order_relaxed) & bit)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) throw std::runtime_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    configured.fetch_or(bit, std::memory_order_relaxed);
  }
  kern<<<grid, PAIR ? DT_THREADS : DT_THREADS_SINGLE, smem, stream>>>(tq, tk, tv, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("dense attention (tcgen05) launch: ") + cudaGetErrorString(e));
}

void launch_dense_attention_tc(const void* q, const void* k, const void* v, void* out, const uint8_t* key_mask,
                               int mask_ld, int B, int Sq, int Sk, int H, int D, const long long* q_strides,
                               const long long* k_strides, const long long* v_strides, float scale,
                               uint32_t* status, cudaStream_t stream) {
  if (B == 0 || Sq == 0) return;
  if (!dense_attention_tc_supported(B, Sq, Sk, H, D, q_strides, k_strides, v_strides))
    throw std::runtime_error("dense attention (tcgen05): unsupported shape or strides");
  if (key_mask != nullptr && (mask_ld % 128 != 0 || mask_ld < Sk || (reinterpret_cast<uintptr_t>(key_mask) & 15) != 0))
    throw std::runtime_error("dense attention (tcgen05): the key mask must be padded to rows of a multiple of 128");
  // a dimension of extent 1 may carry any stride in the view; give TMA the one of a packed tensor
  auto fix = [&](const long long* s, int rows, long long* o) {
    o[1] = s[1];
    o[2] = H > 1 ? s[2] : D;
    o[0] = B > 1 ? s[0] : s[1] * rows;
  };
  long long qs[3], ks[3], vs[3];
  fix(q_strides, Sq, qs);
  fix(k_strides, Sk, ks);
  fix(v_strides, Sk, vs);
  DenseTcParams p{};
  p.out = reinterpret_cast<bf16*>(out);
  p.key_mask = key_mask;
  p.mask_ld = mask_ld;
  p.Sq = Sq;
  p.Sk = Sk;
  p.H = H;
  p.D = D;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  const CUtensorMap tq = dt_tmap(q, B, Sq, H, D, qs);
  const CUtensorMap tk = dt_tmap(k, B, Sk, H, D, ks);
  const CUtensorMap tv = dt_tmap(v, B, Sk, H, D, vs);
  if (D <= 64) {
    // 81 KB of shared memory and 256 columns per CTA: two CTAs per SM
    dt_launch<64, false>(tq, tk, tv, p, dim3((Sq + DT_BM - 1) / DT_BM, H, B), stream);
  } else {
    dt_launch<128, true>(tq, tk, tv, p, dim3((Sq + 2 * DT_BM - 1) / (2 * DT_BM), H, B), stream);
  }
}

}  // namespace fc
