// Python bindings (torch extension `fastcache_b200._C`).  Tensors are checked here
// (device, dtype, contiguity, alignment) so the kernels can assume their layout.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdlib>
#include <mutex>
#include <string>
#include <unordered_map>

#include "gemm.h"
#include "kernels.h"
#include "workspace.h"

namespace {

using torch::Tensor;

struct DeviceWorkspace {
  Tensor gemm_scratch, gemm_counters, grid_sync, attn_o, attn_lse, attn_counters;
  fc::StreamWorkspace raw;
};
struct DeviceState {
  Tensor status;
};
std::unordered_map<uint64_t, DeviceWorkspace> g_ws;      // (device, stream) -> scratch
std::unordered_map<int, DeviceState> g_dev;
std::unordered_map<uint64_t, int> g_stream_sms;
std::mutex g_mu;

using fc::ATTN_COUNTERS;
using fc::ATTN_LSE_FLOATS;
using fc::ATTN_WS_FLOATS;

Tensor& device_status(int dev) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_dev.find(dev);
  if (it != g_dev.end()) return it->second.status;
  DeviceState d;
  d.status = torch::zeros({4}, torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, dev));
  return g_dev.emplace(dev, std::move(d)).first->second.status;
}

DeviceWorkspace& workspace(int dev, cudaStream_t stream) {
  Tensor& status = device_status(dev);
  std::lock_guard<std::mutex> lk(g_mu);
  // stream handles are pointers: fold the device into the bits an aligned pointer leaves free
  const uint64_t key = (reinterpret_cast<uint64_t>(stream) << 8) ^ uint64_t(dev & 0xFF);
  auto it = g_ws.find(key);
  if (it != g_ws.end()) return it->second;
  auto f32 = torch::TensorOptions().dtype(torch::kFloat32).device(torch::kCUDA, dev);
  auto i32 = torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, dev);
  DeviceWorkspace w;
  w.gemm_scratch = torch::empty({int64_t(fc::gemm_scratch_bytes() / 4)}, f32);
  w.gemm_counters = torch::zeros({int64_t(fc::gemm_counter_bytes() / 4)}, i32);
  w.grid_sync = torch::zeros({4}, i32);
  w.attn_o = torch::empty({int64_t(ATTN_WS_FLOATS)}, f32);
  w.attn_lse = torch::empty({int64_t(ATTN_LSE_FLOATS)}, f32);
  w.raw.gemm_scratch = w.gemm_scratch.data_ptr<float>();
  w.raw.gemm_counters = w.gemm_counters.data_ptr<int>();
  w.raw.grid_sync = reinterpret_cast<uint32_t*>(w.grid_sync.data_ptr<int>());
  w.raw.attn_o = w.attn_o.data_ptr<float>();
  w.raw.attn_lse = w.attn_lse.data_ptr<float>();
  w.attn_counters = torch::zeros({int64_t(ATTN_COUNTERS)}, i32);
  w.raw.attn_counters = w.attn_counters.data_ptr<int>();
  w.raw.status = reinterpret_cast<uint32_t*>(status.data_ptr<int>());
  return g_ws.emplace(key, std::move(w)).first->second;
}

// the workspace of the current stream of `dev`
DeviceWorkspace& workspace(int dev) { return workspace(dev, at::cuda::getCurrentCUDAStream(dev)); }

uint32_t* status_ptr(int dev) { return reinterpret_cast<uint32_t*>(device_status(dev).data_ptr<int>()); }

void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name, " must be bf16 (got ", t.scalar_type(), ")");
}

int sm_limit_for(cudaStream_t s) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_stream_sms.find(reinterpret_cast<uint64_t>(s));
  return it == g_stream_sms.end() ? 0 : it->second;
}

// y = act(x @ w.T + bias)
Tensor gemm(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, int64_t act,
            const c10::optional<Tensor>& out_opt) {
  check_bf16(x, "x");
  check_bf16(w, "weight");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2, "gemm expects 2-D operands");
  TORCH_CHECK(x.size(1) == w.size(1), "inner dimensions differ: ", x.size(1), " vs ", w.size(1));
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1, "operands must be row-major (unit inner stride)");
  const int64_t M = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(K % 8 == 0, "K must be a multiple of 8 (16-byte rows for TMA)");
  TORCH_CHECK(x.stride(0) % 8 == 0 && w.stride(0) % 8 == 0, "row pitches must be multiples of 8 elements");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t N_out = (act == fc::ACT_SWIGLU) ? N / 2 : N;      // fused SwiGLU halves the width
  TORCH_CHECK(act != fc::ACT_SWIGLU || (M > 256 && N % 256 == 0), "fused SwiGLU GEMM needs M > 256 and N % 256 == 0");
  Tensor out = out_opt.has_value() ? *out_opt : torch::empty({M, N_out}, x.options());
  check_bf16(out, "out");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == M && out.size(1) == N_out && out.stride(1) == 1, "bad out tensor");
  const void* bptr = nullptr;
  if (bias.has_value() && bias->defined()) {
    check_bf16(*bias, "bias");
    TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "bias must be a contiguous [N] vector");
    bptr = bias->data_ptr();
  }
  if (M == 0) return out;
  auto& ws = workspace(x.get_device());
  fc::GemmWorkspace gw;
  gw.scratch = ws.gemm_scratch.data_ptr<float>();
  gw.counters = ws.gemm_counters.data_ptr<int>();
  gw.status = ws.raw.status;
  gw.grid_sync = ws.raw.grid_sync;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  fc::gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), bptr, int(M), int(N), int(K), x.stride(0), w.stride(0),
                out.stride(0), int(act), gw, sm_limit_for(stream), stream);
  return out;
}

// Launches the GEMM of x @ w.T.  Decode-size inputs may leave fp32 partial sums in the workspace
// instead of a finished result: returns the number of K splits (1 = `out` holds the result).
static int gemm_maybe_partial(const Tensor& x, const Tensor& w, Tensor& out, DeviceWorkspace& ws,
                              cudaStream_t stream) {
  const int64_t M = x.size(0), K = x.size(1), N = w.size(0);
  fc::GemmWorkspace gw;
  gw.scratch = ws.gemm_scratch.data_ptr<float>();
  gw.counters = ws.gemm_counters.data_ptr<int>();
  gw.status = ws.raw.status;
  gw.grid_sync = ws.raw.grid_sync;
  if (M <= 256) {
    return fc::gemm_skinny_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), nullptr, int(M), int(N), int(K),
                                x.stride(0), w.stride(0), out.stride(0), 0, gw, sm_limit_for(stream), 0, false,
                                stream);
  }
  fc::gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), nullptr, int(M), int(N), int(K), x.stride(0),
                w.stride(0), out.stride(0), 0, gw, sm_limit_for(stream), stream);
  return 1;
}

static void check_linear_pair(const Tensor& x, const Tensor& w);

// x @ w.T for a consumer that can reduce split-K partial sums itself: returns the number of K splits.  1: `out`
// holds the bf16 result; > 1: the workspace (`gemm_scratch`) holds fp32 partial sums [splits, M, N] and `out` is
// untouched.
int64_t gemm_partial(const Tensor& x, const Tensor& w, Tensor out) {
  check_linear_pair(x, w);
  check_bf16(out, "out");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == x.size(0) && out.size(1) == w.size(0) && out.stride(1) == 1,
              "bad out tensor");
  if (x.size(0) == 0) return 1;
  c10::cuda::CUDAGuard guard(x.device());
  return gemm_maybe_partial(x, w, out, workspace(x.get_device()), at::cuda::getCurrentCUDAStream());
}

static void check_linear_pair(const Tensor& x, const Tensor& w) {
  check_bf16(x, "x");
  check_bf16(w, "weight");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.size(1) == w.size(1) && x.stride(1) == 1 && w.stride(1) == 1 &&
                  x.size(1) % 8 == 0 && x.stride(0) % 8 == 0 && w.stride(0) % 8 == 0,
              "operands must be row-major bf16 matrices with K % 8 == 0");
}

// residual += x @ w.T (+ bias); returns RMSNorm(residual) * norm_w.  One GEMM launch and one
// norm launch: split-K partial sums are reduced by the norm kernel.
Tensor linear_add_rms_norm(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, Tensor& residual,
                           const Tensor& norm_w, double eps) {
  check_linear_pair(x, w);
  check_bf16(residual, "residual");
  check_bf16(norm_w, "norm weight");
  const int64_t M = x.size(0), N = w.size(0);
  TORCH_CHECK(residual.is_contiguous() && residual.dim() == 2 && residual.size(0) == M && residual.size(1) == N,
              "residual must be contiguous [M, N]");
  TORCH_CHECK(N % 8 == 0 && N <= 8192 && norm_w.numel() == N && norm_w.is_contiguous(), "bad hidden size");
  const void* bptr = nullptr;
  if (bias.has_value() && bias->defined()) {
    check_bf16(*bias, "bias");
    TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "bias must be a contiguous [N] vector");
    bptr = bias->data_ptr();
  }
  c10::cuda::CUDAGuard guard(x.device());
  auto& ws = workspace(x.get_device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  Tensor y = torch::empty({M, N}, x.options());
  if (M == 0) return y;
  if (M <= 256 && fc::fused_epilogues_enabled()) {
    // one kernel: GEMM, grid barrier, then split-K sum + residual add + RMSNorm by the GEMM's own CTAs
    fc::GemmWorkspace gw;
    gw.scratch = ws.raw.gemm_scratch;
    gw.counters = ws.raw.gemm_counters;
    gw.status = ws.raw.status;
    gw.grid_sync = ws.raw.grid_sync;
    fc::SkinnyFused f;
    f.epi = fc::EPI_ADD_NORM;
    f.residual = residual.data_ptr();
    f.norm_w = norm_w.data_ptr();
    f.y = y.data_ptr();
    f.eps = float(eps);
    if (fc::gemm_skinny_bf16(x.data_ptr(), w.data_ptr(), nullptr, bptr, int(M), int(N), int(x.size(1)), x.stride(0),
                             w.stride(0), N, 0, gw, sm_limit_for(stream), 0, false, stream, &f) > 0)
      return y;
  }
  Tensor tmp = torch::empty({M, N}, x.options());
  const int splits = gemm_maybe_partial(x, w, tmp, ws, stream);
  if (splits > 1) {
    fc::launch_add_rms_norm_partials(ws.gemm_scratch.data_ptr<float>(), splits, M * N, bptr, residual.data_ptr(),
                                     norm_w.data_ptr(), y.data_ptr(), M, int(N), float(eps), stream);
  } else {
    if (bptr != nullptr) tmp.add_(*bias);
    fc::launch_rms_norm(tmp.data_ptr(), residual.data_ptr(), norm_w.data_ptr(), y.data_ptr(), M, int(N), float(eps),
                        stream);
  }
  return y;
}

// silu(x @ wg.T) * (x @ wu.T) with w = [wg; wu] stacked on dim 0 ([2 I, K]).
Tensor linear_silu_mul(const Tensor& x, const Tensor& w) {
  check_linear_pair(x, w);
  const int64_t M = x.size(0), N = w.size(0), I = N / 2;
  TORCH_CHECK(N % 16 == 0, "gate|up width must be a multiple of 16");
  c10::cuda::CUDAGuard guard(x.device());
  auto& ws = workspace(x.get_device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  Tensor out = torch::empty({M, I}, x.options());
  if (M == 0) return out;
  if (M <= 128 && N % 256 == 0 && fc::streamk_enabled()) {
    // one persistent kernel: equal spans of (tile, K block) units per SM, gate and up rows share a tile, the owner
    // of a tile adds the other spans' partial sums and applies SwiGLU
    fc::GemmWorkspace gw;
    gw.scratch = ws.raw.gemm_scratch;
    gw.counters = ws.raw.gemm_counters;
    gw.status = ws.raw.status;
    gw.grid_sync = ws.raw.grid_sync;
    if (fc::gemm_streamk_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), nullptr, int(M), int(N), int(x.size(1)),
                              x.stride(0), w.stride(0), I, 0, true, gw, sm_limit_for(stream), stream))
      return out;
  }
  if (M <= 256 && N % 256 == 0 && fc::cluster_splitk_enabled()) {
    // one kernel: gate and up rows share a tile, the K splits reduce inside a cluster, SwiGLU in the epilogue
    fc::GemmWorkspace gw;
    gw.scratch = ws.raw.gemm_scratch;
    gw.counters = ws.raw.gemm_counters;
    gw.status = ws.raw.status;
    gw.grid_sync = ws.raw.grid_sync;
    if (fc::gemm_skinny_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), nullptr, int(M), int(N), int(x.size(1)),
                             x.stride(0), w.stride(0), I, 0, gw, sm_limit_for(stream), 0, false, stream, nullptr,
                             fc::SK_SWIGLU) > 0)
      return out;
  }
  Tensor tmp = torch::empty({M, N}, x.options());
  const int splits = gemm_maybe_partial(x, w, tmp, ws, stream);
  if (splits > 1)
    fc::launch_silu_mul_partials(ws.gemm_scratch.data_ptr<float>(), splits, M * N, out.data_ptr(), M, int(I), stream);
  else
    fc::launch_silu_and_mul(tmp.data_ptr(), out.data_ptr(), M, int(I), stream);
  return out;
}

Tensor rms_norm(const Tensor& x, const Tensor& w, double eps) {
  check_bf16(x, "x");
  check_bf16(w, "weight");
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous(), "rms_norm expects contiguous tensors");
  const int64_t H = x.size(-1);
  TORCH_CHECK(H % 8 == 0 && H <= 8192 && w.numel() == H, "hidden size must be a multiple of 8 and <= 8192");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  fc::launch_rms_norm(x.data_ptr(), nullptr, w.data_ptr(), y.data_ptr(), x.numel() / H, int(H), float(eps),
                      at::cuda::getCurrentCUDAStream());
  return y;
}

Tensor add_rms_norm(const Tensor& x, Tensor& residual, const Tensor& w, double eps) {
  check_bf16(x, "x");
  check_bf16(residual, "residual");
  check_bf16(w, "weight");
  TORCH_CHECK(x.is_contiguous() && residual.is_contiguous() && w.is_contiguous(), "expects contiguous tensors");
  TORCH_CHECK(x.sizes() == residual.sizes(), "x and residual differ in shape");
  const int64_t H = x.size(-1);
  TORCH_CHECK(H % 8 == 0 && H <= 8192 && w.numel() == H, "hidden size must be a multiple of 8 and <= 8192");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  fc::launch_rms_norm(x.data_ptr(), residual.data_ptr(), w.data_ptr(), y.data_ptr(), x.numel() / H, int(H),
                      float(eps), at::cuda::getCurrentCUDAStream());
  return y;
}

Tensor layer_norm(const Tensor& x, const Tensor& w, const Tensor& b, double eps) {
  check_bf16(x, "x");
  check_bf16(w, "weight");
  check_bf16(b, "bias");
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous() && b.is_contiguous(), "expects contiguous tensors");
  const int64_t H = x.size(-1);
  TORCH_CHECK(H % 8 == 0 && H <= 8192 && w.numel() == H && b.numel() == H, "bad hidden size");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  fc::launch_layer_norm(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), x.numel() / H, int(H), float(eps),
                        at::cuda::getCurrentCUDAStream());
  return y;
}

Tensor silu_and_mul(const Tensor& x) {
  check_bf16(x, "x");
  TORCH_CHECK(x.is_contiguous() && x.size(-1) % 16 == 0, "expects contiguous input with last dim % 16 == 0");
  const int64_t I = x.size(-1) / 2;
  auto sizes = x.sizes().vec();
  sizes.back() = I;
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty(sizes, x.options());
  fc::launch_silu_and_mul(x.data_ptr(), y.data_ptr(), x.numel() / (2 * I), int(I), at::cuda::getCurrentCUDAStream());
  return y;
}

Tensor embedding(const Tensor& ids, const Tensor& weight, int64_t vocab_start) {
  check_bf16(weight, "weight");
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == torch::kInt64 && ids.is_contiguous(), "ids must be int64 CUDA");
  TORCH_CHECK(weight.is_contiguous() && weight.size(1) % 8 == 0, "bad embedding table");
  c10::cuda::CUDAGuard guard(weight.device());
  Tensor out = torch::empty({ids.numel(), weight.size(1)}, weight.options());
  fc::launch_embedding(ids.data_ptr(), weight.data_ptr(), out.data_ptr(), int(ids.numel()), int(weight.size(1)),
                       int(weight.size(0)), int(vocab_start), at::cuda::getCurrentCUDAStream());
  return out;
}

Tensor rope_qknorm_store(const Tensor& qkv, const Tensor& positions, const Tensor& cos_sin, int64_t Hq, int64_t Hkv,
                         int64_t D, const c10::optional<Tensor>& q_w, const c10::optional<Tensor>& k_w, double eps,
                         const c10::optional<Tensor>& k_cache, const c10::optional<Tensor>& v_cache,
                         const c10::optional<Tensor>& slots) {
  check_bf16(qkv, "qkv");
  TORCH_CHECK(qkv.is_contiguous() && qkv.dim() == 2 && qkv.size(1) == (Hq + 2 * Hkv) * D, "bad qkv shape");
  TORCH_CHECK(positions.scalar_type() == torch::kInt64 && positions.is_contiguous() && positions.is_cuda(),
              "positions must be int64 CUDA");
  TORCH_CHECK(cos_sin.scalar_type() == torch::kFloat32 && cos_sin.is_contiguous() && cos_sin.size(1) == D &&
                  cos_sin.is_cuda(), "cos_sin must be fp32 [max_pos, D] on the device");
  TORCH_CHECK(D % 8 == 0 && D <= 256, "head_dim must be a multiple of 8 and <= 256");
  const int64_t T = qkv.size(0);
  c10::cuda::CUDAGuard guard(qkv.device());
  Tensor q_out = torch::empty({T, Hq, D}, qkv.options());
  const void *qw = nullptr, *kw = nullptr, *sl = nullptr;
  void *kc = nullptr, *vc = nullptr;
  int64_t num_slots = 0, block_size = 1;
  if (q_w.has_value() && q_w->defined()) { check_bf16(*q_w, "q_norm"); qw = q_w->data_ptr(); }
  if (k_w.has_value() && k_w->defined()) { check_bf16(*k_w, "k_norm"); kw = k_w->data_ptr(); }
  if (k_cache.has_value() && k_cache->defined() && slots.has_value() && slots->defined()) {
    check_bf16(*k_cache, "k_cache");
    check_bf16(*v_cache, "v_cache");
    TORCH_CHECK(k_cache->is_contiguous() && v_cache->is_contiguous(), "cache slices must be contiguous");
    TORCH_CHECK(k_cache->dim() == 4 && k_cache->size(3) == D && k_cache->size(1) == Hkv,
                "cache layout must be [blocks, Hkv, block, D]");
    TORCH_CHECK(slots->scalar_type() == torch::kInt32 && slots->numel() == T && slots->is_cuda(),
                "slot_mapping must be int32 [T]");
    kc = k_cache->data_ptr();
    vc = v_cache->data_ptr();
    sl = slots->data_ptr();
    num_slots = k_cache->size(0) * k_cache->size(2);
    block_size = k_cache->size(2);
  }
  fc::launch_rope_qknorm_store(qkv.data_ptr(), positions.data_ptr(), cos_sin.data_ptr(), qw, kw, q_out.data_ptr(),
                               kc, vc, sl, int(T), int(Hq), int(Hkv), int(D), float(eps), num_slots, int(block_size),
                               status_ptr(qkv.get_device()), at::cuda::getCurrentCUDAStream());
  return q_out;
}

// qkv = x @ w.T, then q/k RMSNorm + rotary + paged K/V store (head_dim 128).  Decode-size GEMMs leave split-K
// partial sums that the rope kernel reduces itself: two launches instead of three.
Tensor linear_rope_qknorm_store(const Tensor& x, const Tensor& w, const Tensor& positions, const Tensor& cos_sin,
                                int64_t Hq, int64_t Hkv, int64_t D, const c10::optional<Tensor>& q_w,
                                const c10::optional<Tensor>& k_w, double eps, const Tensor& k_cache,
                                const Tensor& v_cache, const Tensor& slots) {
  check_linear_pair(x, w);
  const int64_t T = x.size(0), N = w.size(0);
  TORCH_CHECK(D == 128 && N == (Hq + 2 * Hkv) * D, "fused qkv + rope needs head_dim 128 and N = (Hq + 2 Hkv) * 128");
  c10::cuda::CUDAGuard guard(x.device());
  auto& ws = workspace(x.get_device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  Tensor qkv = torch::empty({T, N}, x.options());
  if (T == 0) return torch::empty({0, Hq, D}, x.options());
  const int splits = gemm_maybe_partial(x, w, qkv, ws, stream);
  if (splits <= 1) return rope_qknorm_store(qkv, positions, cos_sin, Hq, Hkv, D, q_w, k_w, eps, k_cache, v_cache, slots);
  TORCH_CHECK(positions.scalar_type() == torch::kInt64 && positions.is_contiguous() && positions.is_cuda(),
              "positions must be int64 CUDA");
  TORCH_CHECK(cos_sin.scalar_type() == torch::kFloat32 && cos_sin.is_contiguous() && cos_sin.size(1) == D &&
                  cos_sin.is_cuda(), "cos_sin must be fp32 [max_pos, D] on the device");
  check_bf16(k_cache, "k_cache");
  check_bf16(v_cache, "v_cache");
  TORCH_CHECK(k_cache.is_contiguous() && v_cache.is_contiguous() && k_cache.dim() == 4 && k_cache.size(3) == D &&
                  k_cache.size(1) == Hkv, "cache layout must be contiguous [blocks, Hkv, block, D]");
  TORCH_CHECK(slots.scalar_type() == torch::kInt32 && slots.numel() == T && slots.is_cuda(),
              "slot_mapping must be int32 [T]");
  const void *qw = nullptr, *kw = nullptr;
  if (q_w.has_value() && q_w->defined()) { check_bf16(*q_w, "q_norm"); qw = q_w->data_ptr(); }
  if (k_w.has_value() && k_w->defined()) { check_bf16(*k_w, "k_norm"); kw = k_w->data_ptr(); }
  Tensor q_out = torch::empty({T, Hq, D}, x.options());
  fc::launch_rope_qknorm_store(nullptr, positions.data_ptr(), cos_sin.data_ptr(), qw, kw, q_out.data_ptr(),
                               k_cache.data_ptr(), v_cache.data_ptr(), slots.data_ptr(), int(T), int(Hq), int(Hkv),
                               int(D), float(eps), k_cache.size(0) * k_cache.size(2), int(k_cache.size(2)),
                               status_ptr(x.get_device()), stream, ws.gemm_scratch.data_ptr<float>(), splits, T * N);
  return q_out;
}

void check_cache(const Tensor& kc, const Tensor& vc, int64_t D) {
  check_bf16(kc, "k_cache");
  check_bf16(vc, "v_cache");
  TORCH_CHECK(kc.dim() == 4 && kc.is_contiguous() && vc.is_contiguous() && kc.size(3) == D,
              "cache layout must be contiguous [blocks, Hkv, block, D]");
}

Tensor prefill_attention(const Tensor& q, const Tensor& kc, const Tensor& vc, const Tensor& block_tables,
                         const Tensor& cu_q, const Tensor& kv_lens, double scale, int64_t max_q_len,
                         int64_t impl) {
  // impl: 0 = choose, 1 = mma.sync kernel, 2 = tcgen05 kernel (one query tile per CTA),
  // 3 = tcgen05 kernel with two query tiles per CTA (what 0 picks for head_dim 128)
  check_bf16(q, "q");
  TORCH_CHECK(q.dim() == 3 && q.is_contiguous(), "q must be contiguous [T, Hq, D]");
  const int64_t Hq = q.size(1), D = q.size(2);
  check_cache(kc, vc, D);
  TORCH_CHECK(block_tables.scalar_type() == torch::kInt32 && block_tables.dim() == 2 && block_tables.is_contiguous(),
              "block_tables must be int32 [B, max_blocks]");
  TORCH_CHECK(cu_q.scalar_type() == torch::kInt32 && kv_lens.scalar_type() == torch::kInt32, "lengths must be int32");
  const int64_t B = kv_lens.numel();
  TORCH_CHECK(cu_q.numel() == B + 1 && block_tables.size(0) >= B, "inconsistent batch metadata");
  if (max_q_len <= 0) max_q_len = q.size(0);
  c10::cuda::CUDAGuard guard(q.device());
  Tensor out = torch::empty_like(q);
  const bool tc_ok = fc::prefill_attention_tc_supported(int(D), int(kc.size(2)));
  TORCH_CHECK((impl != 2 && impl != 3) || tc_ok, "tcgen05 prefill attention needs head_dim 128 and block_size % 8 == 0");
  if (impl == 3 || (impl == 0 && tc_ok && max_q_len > 64)) {
    fc::launch_prefill_attention_tc2(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), block_tables.data_ptr<int>(),
                                     cu_q.data_ptr<int>(), kv_lens.data_ptr<int>(), out.data_ptr(), q.size(0), int(B),
                                     int(max_q_len), int(Hq), int(kc.size(1)), int(kc.size(2)),
                                     int(block_tables.size(1)), int(kc.size(0)), float(scale),
                                     status_ptr(q.get_device()), at::cuda::getCurrentCUDAStream());
    return out;
  }
  if (impl == 2 || (impl == 0 && tc_ok && max_q_len > 64)) {
    fc::launch_prefill_attention_tc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), block_tables.data_ptr<int>(),
                                    cu_q.data_ptr<int>(), kv_lens.data_ptr<int>(), out.data_ptr(), q.size(0), int(B),
                                    int(max_q_len), int(Hq), int(kc.size(1)), int(kc.size(2)),
                                    int(block_tables.size(1)), int(kc.size(0)), float(scale),
                                    status_ptr(q.get_device()), at::cuda::getCurrentCUDAStream());
    return out;
  }
  fc::launch_prefill_attention(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), block_tables.data_ptr<int>(),
                               cu_q.data_ptr<int>(), kv_lens.data_ptr<int>(), out.data_ptr(), int(B), int(max_q_len),
                               int(Hq), int(kc.size(1)), int(D), int(kc.size(2)), int(block_tables.size(1)),
                               int(kc.size(0)), float(scale), status_ptr(q.get_device()),
                               at::cuda::getCurrentCUDAStream());
  return out;
}

// Split-KV decode attention merges its splits in the attention kernel itself (the last split of a (request, KV
// head) to arrive does it) when FC_DECODE_MERGE_KERNEL=0; else the separate merge kernel runs.
static int g_merge_in_kernel = -1;
bool decode_merge_in_kernel() {
  if (g_merge_in_kernel < 0) {
    const char* e = std::getenv("FC_DECODE_MERGE_KERNEL");
    g_merge_in_kernel = (e != nullptr && e[0] == '0') ? 1 : 0;
  }
  return g_merge_in_kernel == 1;
}
void set_decode_merge_in_kernel(bool on) { g_merge_in_kernel = on ? 1 : 0; }

// splits <= 0: choose from the batch shape and `max_ctx`
Tensor decode_attention(const Tensor& q, const Tensor& kc, const Tensor& vc, const Tensor& block_tables,
                        const Tensor& context_lens, double scale, int64_t splits, int64_t max_ctx) {
  check_bf16(q, "q");
  TORCH_CHECK(q.dim() == 3 && q.is_contiguous(), "q must be contiguous [B, Hq, D]");
  const int64_t B = q.size(0), Hq = q.size(1), D = q.size(2);
  check_cache(kc, vc, D);
  const int64_t Hkv = kc.size(1);
  TORCH_CHECK(block_tables.scalar_type() == torch::kInt32 && block_tables.dim() == 2 && block_tables.is_contiguous() &&
                  block_tables.size(0) >= B, "block_tables must be int32 [B, max_blocks]");
  TORCH_CHECK(context_lens.scalar_type() == torch::kInt32 && context_lens.numel() >= B, "context_lens must be int32 [B]");
  c10::cuda::CUDAGuard guard(q.device());
  auto& ws = workspace(q.get_device());
  if (max_ctx <= 0) max_ctx = block_tables.size(1) * kc.size(2);
  if (splits <= 0) splits = fc::decode_attn_pick_splits(int(B), int(Hkv), int(max_ctx), fc::gemm_num_sms());
  while (splits > 1 && (B * Hq * splits * D > ATTN_WS_FLOATS || B * Hq * splits > ATTN_LSE_FLOATS)) --splits;
  Tensor out = torch::empty_like(q);
  fc::launch_decode_attention(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), block_tables.data_ptr<int>(),
                              context_lens.data_ptr<int>(), out.data_ptr(), ws.attn_o.data_ptr<float>(),
                              ws.attn_lse.data_ptr<float>(), int(B), int(Hq), int(Hkv), int(D), int(kc.size(2)),
                              int(block_tables.size(1)), int(kc.size(0)), int(splits), float(scale),
                              status_ptr(q.get_device()), at::cuda::getCurrentCUDAStream(),
                              (decode_merge_in_kernel() && B * Hkv <= ATTN_COUNTERS) ? ws.raw.attn_counters : nullptr);
  return out;
}

// q [B, Sq, H, D], k / v [B, Sk, H, D]; any strides with a contiguous last dim; key_mask [B, Sk] bool.
// impl: 0 = the tcgen05 kernel where the strides can be described to TMA, else the mma.sync kernel; 1 = mma.sync;
// 2 = tcgen05 (raises when it cannot run).
Tensor dense_attention(const Tensor& q, const Tensor& k, const Tensor& v, double scale,
                       const c10::optional<Tensor>& key_mask, int64_t impl) {
  check_bf16(q, "q");
  check_bf16(k, "k");
  check_bf16(v, "v");
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "dense attention expects [B, S, H, D] tensors");
  TORCH_CHECK(q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1, "last dim must be contiguous");
  const int64_t B = q.size(0), Sq = q.size(1), H = q.size(2), D = q.size(3), Sk = k.size(1);
  TORCH_CHECK(k.size(0) == B && v.size(0) == B && k.size(2) == H && v.size(2) == H && k.size(3) == D &&
                  v.size(3) == D && v.size(1) == Sk, "q / k / v shapes do not agree");
  for (const Tensor* t : {&q, &k, &v}) {
    TORCH_CHECK(reinterpret_cast<uintptr_t>(t->data_ptr()) % 16 == 0 && t->stride(0) % 8 == 0 &&
                    t->stride(1) % 8 == 0 && t->stride(2) % 8 == 0, "operands must be 16-byte aligned per row");
  }
  const bool has_mask = key_mask.has_value() && key_mask->defined();
  if (has_mask)
    TORCH_CHECK(key_mask->scalar_type() == torch::kBool && key_mask->dim() == 2 && key_mask->size(0) == B &&
                    key_mask->size(1) == Sk && key_mask->is_cuda(), "key_mask must be bool [B, Sk] on the device");
  c10::cuda::CUDAGuard guard(q.device());
  Tensor out = torch::empty({B, Sq, H, D}, q.options());
  const long long qs[3] = {q.stride(0), q.stride(1), q.stride(2)};
  const long long ks[3] = {k.stride(0), k.stride(1), k.stride(2)};
  const long long vs[3] = {v.stride(0), v.stride(1), v.stride(2)};
  const bool tc_ok = B > 0 && Sq > 0 &&
                     fc::dense_attention_tc_supported(int(B), int(Sq), int(Sk), int(H), int(D), qs, ks, vs);
  TORCH_CHECK(impl != 2 || tc_ok || B == 0 || Sq == 0, "dense attention: the tcgen05 kernel cannot take these strides");
  auto stream = at::cuda::getCurrentCUDAStream();
  if (impl != 1 && tc_ok) {
    const uint8_t* mask = nullptr;
    Tensor mask_p;
    const int64_t ld = (Sk + 127) / 128 * 128;
    if (has_mask) {
      mask_p = torch::zeros({B, ld}, key_mask->options().dtype(torch::kUInt8));
      mask_p.narrow(1, 0, Sk).copy_(*key_mask);
      mask = reinterpret_cast<const uint8_t*>(mask_p.data_ptr());
    }
    fc::launch_dense_attention_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), mask, int(ld), int(B),
                                  int(Sq), int(Sk), int(H), int(D), qs, ks, vs, float(scale),
                                  status_ptr(q.get_device()), stream);
    return out;
  }
  const uint8_t* mask = nullptr;
  Tensor mask_c;
  if (has_mask) {
    mask_c = key_mask->contiguous();
    mask = reinterpret_cast<const uint8_t*>(mask_c.data_ptr());
  }
  fc::launch_dense_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), mask, int(B), int(Sq),
                             int(Sk), int(H), int(D), qs, ks, vs, float(scale), stream);
  return out;
}

// Tokens [B] (with_status false) or [B + 1]: the tokens followed by the device status code, which the host then
// gets with the tokens it reads back anyway.  Column j of the logits is vocabulary entry vocab_offset + j;
// entries >= v_limit (-1: none) are padding.
Tensor sample(const Tensor& logits, const Tensor& temps, int64_t seed, bool with_status, int64_t vocab_offset,
              int64_t v_limit) {
  check_bf16(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "logits must be [B, V] with unit inner stride");
  TORCH_CHECK(temps.is_cuda() && temps.scalar_type() == torch::kFloat32 && temps.numel() == logits.size(0),
              "temperatures must be fp32 [B] on the device");
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t B = logits.size(0);
  Tensor out = torch::empty({B + (with_status ? 1 : 0)}, logits.options().dtype(torch::kInt64));
  if (B == 0 && with_status) out.zero_();
  fc::launch_sample(logits.data_ptr(), temps.data_ptr(), out.data_ptr(), int(B), int(logits.size(1)),
                    logits.stride(0), uint32_t(seed), at::cuda::getCurrentCUDAStream(), int(vocab_offset),
                    int(v_limit), with_status ? status_ptr(logits.get_device()) : nullptr);
  return out;
}

// Reads the code bits of the device status word and clears them (synchronises the current stream); the wait
// limit kept in the upper bits stays.
int64_t read_status(int64_t device) {
  Tensor& st = device_status(int(device));
  const int64_t v = st[0].item<int>();
  if ((v & 0xFF) != 0) st[0].bitwise_and_(~0xFF);
  return v & 0xFF;
}

// Limit of every bounded device wait (mbarriers and flags of other GPUs) in microseconds for kernels that get this
// device's status word; 0 restores the built-in limits.  For tests and for deployments that prefer to fail fast.
void set_wait_limit_us(int64_t device, int64_t us) {
  TORCH_CHECK(us >= 0 && us < (1 << 24), "limit must be in [0, 2^24) microseconds");
  Tensor& st = device_status(int(device));
  const int64_t v = st[0].item<int>();
  st[0].fill_(int64_t(int32_t((uint32_t(v) & 0xFFu) | (uint32_t(us) << 8))));
}

// After a kernel reported a wait that ran out, the arrival counters it was using may be left mid-count: zero the
// grid-barrier words and the split-K tile counters of every stream of the device (the host calls this once the
// device is idle, e.g. from LLMEngine.recover()).
void reset_sync_state(int64_t device) {
  std::lock_guard<std::mutex> lk(g_mu);
  c10::cuda::CUDAGuard guard(c10::Device(c10::kCUDA, int(device)));
  cudaDeviceSynchronize();
  for (auto& kv : g_ws) {
    if (int(kv.first & 0xFF) != int(device & 0xFF)) continue;
    // plain memsets on the raw pointers: the tensors may have been created under inference mode
    cudaMemset(kv.second.raw.grid_sync, 0, 4 * sizeof(int));
    cudaMemset(kv.second.raw.gemm_counters, 0, fc::gemm_counter_bytes());
    cudaMemset(kv.second.raw.attn_counters, 0, size_t(ATTN_COUNTERS) * sizeof(int));
  }
}

void register_stream_sms(int64_t stream_ptr, int64_t sms) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (sms <= 0) g_stream_sms.erase(uint64_t(stream_ptr));
  else g_stream_sms[uint64_t(stream_ptr)] = int(sms);
}

}  // namespace

void register_greenctx(pybind11::module_& m);
void register_compress(pybind11::module_& m);
void register_comm(pybind11::module_& m);
void register_symm(pybind11::module_& m);

namespace fc {
const StreamWorkspace& stream_workspace(int device, cudaStream_t stream) { return workspace(device, stream).raw; }
int stream_sm_limit(cudaStream_t stream) { return sm_limit_for(stream); }
static int g_fused_epilogues = -1;     // -1: take the environment variable
bool fused_epilogues_enabled() {
  if (g_fused_epilogues < 0) {
    // off unless asked for: measured on B200, the pair of kernels chained by programmatic dependent launch is
    // faster (the second kernel of the pair needs no shared memory, so the GEMM after it is already resident and
    // has its first weight tiles in flight while the reduction runs; the one-kernel form keeps the SM's shared
    // memory until the reduction is done)
    const char* e = std::getenv("FC_FUSED_EPILOGUE");
    g_fused_epilogues = (e != nullptr && std::string(e) == "1") ? 1 : 0;
  }
  return g_fused_epilogues == 1;
}
void set_fused_epilogues(bool on) { g_fused_epilogues = on ? 1 : 0; }
}  // namespace fc

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, "y = act(x @ w.T + bias) on tcgen05", py::arg("x"), py::arg("w"), py::arg("bias") = py::none(),
        py::arg("act") = 0, py::arg("out") = py::none());
  m.def("linear_add_rms_norm", &linear_add_rms_norm);
  m.def("linear_silu_mul", &linear_silu_mul);
  m.def("rms_norm", &rms_norm);
  m.def("add_rms_norm", &add_rms_norm);
  m.def("layer_norm", &layer_norm);
  m.def("silu_and_mul", &silu_and_mul);
  m.def("embedding", &embedding);
  m.def("rope_qknorm_store", &rope_qknorm_store);
  m.def("linear_rope_qknorm_store", &linear_rope_qknorm_store);
  m.def("gemm_partial", &gemm_partial);
  m.def("gemm_scratch", [](int64_t device) { return workspace(int(device)).gemm_scratch; },
        "split-K scratch of the CURRENT stream of the device");
  m.def("prefill_attention", &prefill_attention);
  m.def("set_decode_merge_in_kernel", &set_decode_merge_in_kernel);
  m.def("decode_merge_in_kernel", &decode_merge_in_kernel);
  m.def("decode_attention", &decode_attention, py::arg("q"), py::arg("k_cache"), py::arg("v_cache"),
        py::arg("block_tables"), py::arg("context_lens"), py::arg("scale"), py::arg("splits") = 0,
        py::arg("max_ctx") = 0);
  m.def("sample", &sample, py::arg("logits"), py::arg("temperatures"), py::arg("seed"), py::arg("with_status") = false,
        py::arg("vocab_offset") = 0, py::arg("v_limit") = -1);
  m.def("dense_attention", &dense_attention, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("scale"),
        py::arg("key_mask") = py::none(), py::arg("impl") = 0);
  m.def("read_status", &read_status);
  m.def("set_wait_limit_us", &set_wait_limit_us);
  m.def("reset_sync_state", &reset_sync_state);
  m.def("set_fused_epilogues", &fc::set_fused_epilogues, "one-kernel GEMM + (all-reduce +) add + RMSNorm for decode sizes");
  m.def("fused_epilogues_enabled", &fc::fused_epilogues_enabled);
  m.def("set_cluster_splitk", &fc::set_cluster_splitk, "split-K of decode-size GEMMs inside thread-block clusters");
  m.def("cluster_splitk_enabled", &fc::cluster_splitk_enabled);
  m.def("set_streamk", &fc::set_streamk, "persistent stream-K form of the decode-size GEMMs with finished outputs");
  m.def("set_gemm_pairs", &fc::set_gemm_pairs, "prefill-size GEMMs as tcgen05.mma.cta_group::2 on CTA pairs");
  m.def("gemm_pairs_mode", &fc::gemm_pairs_mode);
  m.def("streamk_enabled", &fc::streamk_enabled);
  m.def("streamk_mode", &fc::streamk_mode);
  m.def("register_stream_sms", &register_stream_sms);
  m.def("num_sms", []() { return fc::gemm_num_sms(); });
  m.def("status_tensor", [](int64_t device) { return device_status(int(device)); });
  register_greenctx(m);
  register_compress(m);
  register_comm(m);
  register_symm(m);
}
