// Bindings of the fused communication kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <vector>

#include "comm.h"
#include "gemm.h"
#include "workspace.h"

namespace {
using torch::Tensor;

struct CommState {
  bool ready = false;
  fc::CommPeers peers{};
  uint64_t mc[2] = {0, 0};
  Tensor epochs;
  bool sample_ready = false;
  fc::SamplePeers cand{};
};
CommState g_comm;

// slot_rows > 0: the staging buffers hold `world` slots of `slot_rows` rows and the one-shot all-reduce runs in
// its push form (comm.cu)
void comm_init(int64_t rank, int64_t world, const std::vector<int64_t>& data0, const std::vector<int64_t>& data1,
               const std::vector<int64_t>& flags, int64_t mc0, int64_t mc1, int64_t device, int64_t slot_rows,
               int64_t reduced_row0) {
  TORCH_CHECK(world >= 2 && world <= fc::COMM_MAX_WORLD, "world size must be in [2, ", fc::COMM_MAX_WORLD, "]");
  TORCH_CHECK((int64_t)data0.size() == world && (int64_t)data1.size() == world && (int64_t)flags.size() == world,
              "need one pointer per rank");
  g_comm.peers.world = int(world);
  g_comm.peers.rank = int(rank);
  g_comm.peers.slot_rows = int(slot_rows);
  // the two-shot form needs the multicast addresses of both staging buffers
  g_comm.peers.reduced_row0 = (mc0 != 0 && mc1 != 0) ? int(reduced_row0) : 0;
  TORCH_CHECK(slot_rows == 0 || reduced_row0 == 0, "choose one form of the one-shot all-reduce");
  for (int i = 0; i < world; ++i) {
    g_comm.peers.data[0][i] = reinterpret_cast<__nv_bfloat16*>(data0[i]);
    g_comm.peers.data[1][i] = reinterpret_cast<__nv_bfloat16*>(data1[i]);
    g_comm.peers.flags[i] = reinterpret_cast<uint32_t*>(flags[i]);
  }
  g_comm.mc[0] = uint64_t(mc0);
  g_comm.mc[1] = uint64_t(mc1);
  g_comm.epochs = torch::zeros({fc::COMM_MAX_SLOTS},
                               torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, int(device)));
  g_comm.ready = true;
}

void comm_shutdown() {
  g_comm.ready = false;
  g_comm.sample_ready = false;
  g_comm.epochs = Tensor();
}

// Candidate tables (one symmetric allocation of fc::SAMPLE_CELLS_PER_RANK int64 cells per rank, zeroed).
void sample_exchange_init(const std::vector<int64_t>& cells) {
  TORCH_CHECK(g_comm.ready, "comm_init was not called");
  TORCH_CHECK((int64_t)cells.size() == g_comm.peers.world, "need one pointer per rank");
  for (int i = 0; i < g_comm.peers.world; ++i) g_comm.cand.cells[i] = reinterpret_cast<uint64_t*>(cells[i]);
  g_comm.sample_ready = true;
}

// Tokens drawn from vocabulary-sharded logits; every rank returns the same [B] tokens followed by its device
// status code ([B + 1] int64).
Tensor sample_exchange(const Tensor& logits, const Tensor& temps, int64_t seed, int64_t vocab_offset, int64_t v_limit,
                       Tensor status) {
  TORCH_CHECK(g_comm.ready && g_comm.sample_ready, "sample_exchange_init was not called");
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == torch::kBFloat16 && logits.dim() == 2 &&
                  logits.stride(1) == 1, "logits must be bf16 [B, V] with unit inner stride");
  TORCH_CHECK(temps.is_cuda() && temps.scalar_type() == torch::kFloat32 && temps.numel() == logits.size(0),
              "temperatures must be fp32 [B] on the device");
  TORCH_CHECK(logits.size(0) <= fc::COMM_MAX_SLOTS, "at most ", fc::COMM_MAX_SLOTS, " requests per call");
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor out = torch::empty({logits.size(0) + 1}, logits.options().dtype(torch::kInt64));
  fc::launch_sample_exchange(g_comm.peers, g_comm.cand, logits.data_ptr(), temps.data_ptr(), out.data_ptr(),
                             int(logits.size(0)), int(logits.size(1)), logits.stride(0), uint32_t(seed),
                             int(vocab_offset), int(v_limit),
                             reinterpret_cast<uint32_t*>(g_comm.epochs.data_ptr<int>()),
                             reinterpret_cast<uint32_t*>(status.data_ptr<int>()), at::cuda::getCurrentCUDAStream());
  return out;
}

// The partial sums of this rank are rows [0, T) of staging buffer `buf`.  Returns the normalised
// rows; `residual` is updated in place.
Tensor allreduce_add_rmsnorm(int64_t buf, Tensor residual, const Tensor& weight, double eps, bool use_multimem,
                             Tensor status, const c10::optional<Tensor>& partial, int64_t splits,
                             const c10::optional<Tensor>& bias) {
  TORCH_CHECK(g_comm.ready, "comm_init was not called");
  TORCH_CHECK(residual.is_cuda() && residual.scalar_type() == torch::kBFloat16 && residual.is_contiguous() &&
                  residual.dim() == 2, "residual must be contiguous bf16 [T, H]");
  TORCH_CHECK(weight.scalar_type() == torch::kBFloat16 && weight.is_contiguous() && weight.numel() == residual.size(1),
              "bad norm weight");
  TORCH_CHECK(buf == 0 || buf == 1, "buf must be 0 or 1");
  c10::cuda::CUDAGuard guard(residual.device());
  Tensor out = torch::empty_like(residual);
  const void* mc = ((use_multimem || g_comm.peers.reduced_row0 > 0) && g_comm.mc[buf] != 0)
                       ? reinterpret_cast<const void*>(g_comm.mc[buf]) : nullptr;
  const float* part = nullptr;
  const void* bptr = nullptr;
  if (partial.has_value() && partial->defined() && splits > 1) {
    TORCH_CHECK(partial->is_cuda() && partial->scalar_type() == torch::kFloat32 && partial->is_contiguous() &&
                    partial->numel() >= splits * residual.numel(), "partial sums must be fp32 [splits, T, H]");
    part = partial->data_ptr<float>();
    if (bias.has_value() && bias->defined()) {
      TORCH_CHECK(bias->scalar_type() == torch::kBFloat16 && bias->is_contiguous() && bias->numel() == residual.size(1),
                  "bias must be a contiguous bf16 [H] vector");
      bptr = bias->data_ptr();
    }
  }
  fc::launch_allreduce_add_rmsnorm(g_comm.peers, int(buf), mc, residual.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                   int(residual.size(0)), int(residual.size(1)), float(eps),
                                   reinterpret_cast<uint32_t*>(g_comm.epochs.data_ptr<int>()),
                                   reinterpret_cast<uint32_t*>(status.data_ptr<int>()), mc != nullptr,
                                   at::cuda::getCurrentCUDAStream(), part, int(splits), residual.numel(), bptr);
  return out;
}
// Decode-size row-parallel projection with everything that follows it: residual += sum over ranks of (x @ w.T
// (+ bias)); returns RMSNorm(residual) * norm_w.  One kernel when the shape allows (the GEMM's CTAs meet at a grid
// barrier, finish their token rows into staging buffer `buf`, exchange flags with the peers and reduce), else the
// GEMM and the one-shot all-reduce kernel.
Tensor linear_allreduce_add_rmsnorm(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, int64_t buf,
                                    Tensor residual, const Tensor& norm_w, double eps, bool use_multimem,
                                    Tensor status) {
  TORCH_CHECK(g_comm.ready, "comm_init was not called");
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.dim() == 2 && x.stride(1) == 1 &&
                  x.stride(0) % 8 == 0 && x.size(1) % 8 == 0, "x must be a row-major bf16 matrix with K % 8 == 0");
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == torch::kBFloat16 && w.dim() == 2 && w.stride(1) == 1 &&
                  w.stride(0) % 8 == 0 && w.size(1) == x.size(1), "weight must be row-major bf16 [N, K]");
  const int64_t M = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(M <= 256, "decode-size inputs only (at most 256 rows)");
  TORCH_CHECK(residual.is_cuda() && residual.scalar_type() == torch::kBFloat16 && residual.is_contiguous() &&
                  residual.dim() == 2 && residual.size(0) == M && residual.size(1) == N,
              "residual must be contiguous bf16 [M, N]");
  TORCH_CHECK(norm_w.scalar_type() == torch::kBFloat16 && norm_w.is_contiguous() && norm_w.numel() == N,
              "bad norm weight");
  TORCH_CHECK(buf == 0 || buf == 1, "buf must be 0 or 1");
  const void* bptr = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->scalar_type() == torch::kBFloat16 && bias->is_contiguous() && bias->numel() == N,
                "bias must be a contiguous bf16 [N] vector");
    bptr = bias->data_ptr();
  }
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty_like(residual);
  if (M == 0) return out;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const fc::StreamWorkspace& sw = fc::stream_workspace(x.get_device(), stream);
  fc::GemmWorkspace gw;
  gw.scratch = sw.gemm_scratch;
  gw.counters = sw.gemm_counters;
  gw.status = reinterpret_cast<uint32_t*>(status.data_ptr<int>());
  gw.grid_sync = sw.grid_sync;
  const void* mc = ((use_multimem || g_comm.peers.reduced_row0 > 0) && g_comm.mc[buf] != 0)
                       ? reinterpret_cast<const void*>(g_comm.mc[buf]) : nullptr;
  uint32_t* epochs = reinterpret_cast<uint32_t*>(g_comm.epochs.data_ptr<int>());
  const int sm_limit = fc::stream_sm_limit(stream);
  if (fc::fused_epilogues_enabled() && g_comm.peers.slot_rows == 0 && g_comm.peers.reduced_row0 == 0) {
    fc::SkinnyFused f;
    f.epi = fc::EPI_AR_ADD_NORM;
    f.residual = residual.data_ptr();
    f.norm_w = norm_w.data_ptr();
    f.y = out.data_ptr();
    f.eps = float(eps);
    f.peers = &g_comm.peers;
    f.buf = int(buf);
    f.mc_in = mc;
    f.epochs = epochs;
    if (fc::gemm_skinny_bf16(x.data_ptr(), w.data_ptr(), nullptr, bptr, int(M), int(N), int(K), x.stride(0),
                             w.stride(0), N, 0, gw, sm_limit, 0, false, stream, &f) > 0)
      return out;
  }
  // two kernels: the GEMM leaves bf16 rows in the staging buffer or fp32 split-K partial sums in scratch, the
  // all-reduce kernel finishes them
  // (push form: the rank's own slot of its own buffer)
  void* staging = g_comm.peers.data[buf][g_comm.peers.rank] +
                  (size_t)g_comm.peers.rank * g_comm.peers.slot_rows * size_t(N);
  const int splits = fc::gemm_skinny_bf16(x.data_ptr(), w.data_ptr(), staging, bptr, int(M), int(N), int(K),
                                          x.stride(0), w.stride(0), N, 0, gw, sm_limit, 0, false, stream);
  fc::launch_allreduce_add_rmsnorm(g_comm.peers, int(buf), mc, residual.data_ptr(), norm_w.data_ptr(),
                                   out.data_ptr(), int(M), int(N), float(eps), epochs, gw.status, mc != nullptr,
                                   stream, splits > 1 ? sw.gemm_scratch : nullptr, splits, M * N,
                                   splits > 1 ? bptr : nullptr);
  return out;
}

// ------------------------------------------------------------ prefill-size fused GEMM + collective
struct TpState {
  bool ready = false;
  fc::TpBuffers b;
  Tensor owner_done, group_done;
  int64_t stage_rows = 0, xg_rows = 0, hidden = 0;
};
TpState g_tp;

// `flags`: per rank 2 * COMM_MAX_WORLD words (chunk flags) followed by max_groups * COMM_MAX_WORLD words (row-group
// flags of the pipelined reduce-scatter; max_groups = 0: none)
void tp_init(int64_t rank, int64_t world, const std::vector<int64_t>& stage, const std::vector<int64_t>& xg,
             const std::vector<int64_t>& flags, int64_t stage_rows, int64_t xg_rows, int64_t hidden,
             int64_t device, int64_t max_groups, int64_t stage_mc, int64_t xg_mc) {
  TORCH_CHECK(world >= 2 && world <= fc::COMM_MAX_WORLD, "world size must be in [2, ", fc::COMM_MAX_WORLD, "]");
  TORCH_CHECK((int64_t)stage.size() == world && (int64_t)xg.size() == world && (int64_t)flags.size() == world,
              "need one pointer per rank");
  g_tp.b.world = int(world);
  g_tp.b.rank = int(rank);
  for (int i = 0; i < world; ++i) {
    g_tp.b.stage[i] = reinterpret_cast<__nv_bfloat16*>(stage[i]);
    g_tp.b.xg[i] = reinterpret_cast<__nv_bfloat16*>(xg[i]);
    g_tp.b.rs_flags[i] = reinterpret_cast<uint32_t*>(flags[i]);
    g_tp.b.gathered_flags[i] = reinterpret_cast<uint32_t*>(flags[i]) + fc::COMM_MAX_WORLD;
    g_tp.b.group_flags[i] = max_groups > 0 ? reinterpret_cast<uint32_t*>(flags[i]) + 2 * fc::COMM_MAX_WORLD : nullptr;
  }
  g_tp.b.max_groups = int(max_groups);
  g_tp.b.stage_mc = reinterpret_cast<const __nv_bfloat16*>(stage_mc);
  g_tp.b.xg_mc = reinterpret_cast<__nv_bfloat16*>(xg_mc);
  g_tp.b.group_done = nullptr;
  if (max_groups > 0) {
    g_tp.group_done = torch::zeros({fc::COMM_MAX_WORLD * max_groups},
                                   torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, int(device)));
    g_tp.b.group_done = g_tp.group_done.data_ptr<int>();
  }
  g_tp.owner_done = torch::zeros({fc::COMM_MAX_WORLD + 1},
                                 torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, int(device)));
  g_tp.b.owner_done = g_tp.owner_done.data_ptr<int>();
  g_tp.stage_rows = stage_rows;      // rows per source slot of the staging buffer
  g_tp.xg_rows = xg_rows;
  g_tp.hidden = hidden;
  g_tp.ready = true;
}

void check_gemm_operand(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.dim() == 2 && t.stride(1) == 1 &&
                  t.stride(0) % 8 == 0 && t.size(1) % 8 == 0, name, " must be a row-major bf16 matrix with K % 8 == 0");
}

// Partial products of x @ w.T are reduce-scattered, added to `residual` (the rows this rank owns,
// updated in place) and normalised; the normalised rows of every rank land in xg on every rank.
void gemm_rs_add_norm(const Tensor& x, const Tensor& w, Tensor residual, const Tensor& norm_w, double eps,
                      int64_t chunk_rows, int64_t epoch, Tensor status, int64_t sm_limit) {
  TORCH_CHECK(g_tp.ready, "tp_init was not called");
  check_gemm_operand(x, "x");
  check_gemm_operand(w, "weight");
  const int64_t M = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K && N == g_tp.hidden, "weight shape does not match the staging buffers");
  TORCH_CHECK(chunk_rows % 128 == 0 && chunk_rows <= g_tp.stage_rows && M <= g_tp.xg_rows &&
                  chunk_rows * g_tp.b.world >= M, "chunk_rows / token count exceed the staging buffers");
  const int64_t own = std::max<int64_t>(0, std::min<int64_t>(M - g_tp.b.rank * chunk_rows, chunk_rows));
  TORCH_CHECK(residual.scalar_type() == torch::kBFloat16 && residual.is_contiguous() && residual.dim() == 2 &&
                  residual.size(0) == own && residual.size(1) == N, "residual must hold the ", own,
              " rows owned by this rank");
  TORCH_CHECK(norm_w.scalar_type() == torch::kBFloat16 && norm_w.is_contiguous() && norm_w.numel() == N,
              "bad norm weight");
  c10::cuda::CUDAGuard guard(x.device());
  fc::gemm_rs_add_norm(x.data_ptr(), w.data_ptr(), int(M), int(N), int(K), x.stride(0), w.stride(0), g_tp.b,
                       residual.data_ptr(), norm_w.data_ptr(), float(eps), int(chunk_rows), uint32_t(epoch),
                       reinterpret_cast<uint32_t*>(status.data_ptr<int>()), int(sm_limit),
                       at::cuda::getCurrentCUDAStream());
}

// y = xg[:M] @ w.T where xg is this rank's gathered-activation buffer (passed as a tensor view).
Tensor gemm_after_gather(const Tensor& xg_view, const Tensor& w, int64_t chunk_rows, int64_t epoch, Tensor status,
                         int64_t sm_limit, bool swiglu) {
  TORCH_CHECK(g_tp.ready, "tp_init was not called");
  check_gemm_operand(xg_view, "xg");
  check_gemm_operand(w, "weight");
  TORCH_CHECK(xg_view.is_contiguous() && xg_view.data_ptr() == g_tp.b.xg[g_tp.b.rank],
              "xg must be the gathered-activation buffer of this rank");
  const int64_t M = xg_view.size(0), K = xg_view.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K, "inner dimensions differ");
  c10::cuda::CUDAGuard guard(w.device());
  TORCH_CHECK(!swiglu || N % 256 == 0, "fused SwiGLU needs N % 256 == 0");
  Tensor out = torch::empty({M, swiglu ? N / 2 : N}, w.options());
  fc::gemm_after_gather(xg_view.data_ptr(), w.data_ptr(), out.data_ptr(), int(M), int(N), int(K), w.stride(0),
                        out.stride(0), g_tp.b, int(chunk_rows), uint32_t(epoch),
                        reinterpret_cast<uint32_t*>(status.data_ptr<int>()), int(sm_limit),
                        at::cuda::getCurrentCUDAStream(), swiglu);
  return out;
}

void wait_gathered(int64_t epoch, Tensor status) {
  TORCH_CHECK(g_tp.ready, "tp_init was not called");
  fc::wait_gathered(g_tp.b, uint32_t(epoch), reinterpret_cast<uint32_t*>(status.data_ptr<int>()),
                    at::cuda::getCurrentCUDAStream());
}
}  // namespace

void register_comm(pybind11::module_& m) {
  m.def("comm_init", &comm_init, pybind11::arg("rank"), pybind11::arg("world"), pybind11::arg("data0"),
        pybind11::arg("data1"), pybind11::arg("flags"), pybind11::arg("mc0"), pybind11::arg("mc1"),
        pybind11::arg("device"), pybind11::arg("slot_rows") = 0, pybind11::arg("reduced_row0") = 0);
  m.def("comm_shutdown", &comm_shutdown);
  m.def("sample_exchange_init", &sample_exchange_init);
  m.def("sample_exchange", &sample_exchange);
  m.def("sample_cells_per_rank", []() { return int64_t(fc::SAMPLE_CELLS_PER_RANK); });
  m.def("allreduce_add_rmsnorm", &allreduce_add_rmsnorm, pybind11::arg("buf"), pybind11::arg("residual"),
        pybind11::arg("weight"), pybind11::arg("eps"), pybind11::arg("use_multimem"), pybind11::arg("status"),
        pybind11::arg("partial") = pybind11::none(), pybind11::arg("splits") = 0,
        pybind11::arg("bias") = pybind11::none());
  m.def("linear_allreduce_add_rmsnorm", &linear_allreduce_add_rmsnorm);
  m.def("tp_init", &tp_init, pybind11::arg("rank"), pybind11::arg("world"), pybind11::arg("stage"), pybind11::arg("xg"),
        pybind11::arg("flags"), pybind11::arg("stage_rows"), pybind11::arg("xg_rows"), pybind11::arg("hidden"),
        pybind11::arg("device"), pybind11::arg("max_groups") = 0, pybind11::arg("stage_mc") = 0,
        pybind11::arg("xg_mc") = 0);
  m.def("set_tp_nvls", &fc::set_tp_nvls, "pipelined row-parallel GEMM: sums and broadcasts through NVSwitch multicast");
  m.def("tp_nvls_enabled", &fc::tp_nvls_enabled);
  m.def("set_tp_pipeline", &fc::set_tp_pipeline, "row-parallel prefill GEMM: reduce row groups while the GEMM runs");
  m.def("tp_pipeline_enabled", &fc::tp_pipeline_enabled);
  m.def("gemm_rs_add_norm", &gemm_rs_add_norm);
  m.def("gemm_after_gather", &gemm_after_gather, pybind11::arg("xg"), pybind11::arg("weight"),
        pybind11::arg("chunk_rows"), pybind11::arg("epoch"), pybind11::arg("status"), pybind11::arg("sm_limit"),
        pybind11::arg("swiglu") = false);
  m.def("wait_gathered", &wait_gathered);
}
