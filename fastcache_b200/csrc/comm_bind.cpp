// Bindings of the fused communication kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <vector>

#include "comm.h"

namespace {
using torch::Tensor;

struct CommState {
  bool ready = false;
  fc::CommPeers peers{};
  uint64_t mc[2] = {0, 0};
  Tensor epochs;
};
CommState g_comm;

void comm_init(int64_t rank, int64_t world, const std::vector<int64_t>& data0, const std::vector<int64_t>& data1,
               const std::vector<int64_t>& flags, int64_t mc0, int64_t mc1, int64_t device) {
  TORCH_CHECK(world >= 2 && world <= fc::COMM_MAX_WORLD, "world size must be in [2, ", fc::COMM_MAX_WORLD, "]");
  TORCH_CHECK((int64_t)data0.size() == world && (int64_t)data1.size() == world && (int64_t)flags.size() == world,
              "need one pointer per rank");
  g_comm.peers.world = int(world);
  g_comm.peers.rank = int(rank);
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
  g_comm.epochs = Tensor();
}

// The partial sums of this rank are rows [0, T) of staging buffer `buf`.  Returns the normalised
// rows; `residual` is updated in place.
Tensor allreduce_add_rmsnorm(int64_t buf, Tensor residual, const Tensor& weight, double eps, bool use_multimem,
                             Tensor status) {
  TORCH_CHECK(g_comm.ready, "comm_init was not called");
  TORCH_CHECK(residual.is_cuda() && residual.scalar_type() == torch::kBFloat16 && residual.is_contiguous() &&
                  residual.dim() == 2, "residual must be contiguous bf16 [T, H]");
  TORCH_CHECK(weight.scalar_type() == torch::kBFloat16 && weight.is_contiguous() && weight.numel() == residual.size(1),
              "bad norm weight");
  TORCH_CHECK(buf == 0 || buf == 1, "buf must be 0 or 1");
  c10::cuda::CUDAGuard guard(residual.device());
  Tensor out = torch::empty_like(residual);
  const void* mc = (use_multimem && g_comm.mc[buf] != 0) ? reinterpret_cast<const void*>(g_comm.mc[buf]) : nullptr;
  fc::launch_allreduce_add_rmsnorm(g_comm.peers, int(buf), mc, residual.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                   int(residual.size(0)), int(residual.size(1)), float(eps),
                                   reinterpret_cast<uint32_t*>(g_comm.epochs.data_ptr<int>()),
                                   reinterpret_cast<uint32_t*>(status.data_ptr<int>()), mc != nullptr,
                                   at::cuda::getCurrentCUDAStream());
  return out;
}
}  // namespace

void register_comm(pybind11::module_& m) {
  m.def("comm_init", &comm_init);
  m.def("comm_shutdown", &comm_shutdown);
  m.def("allreduce_add_rmsnorm", &allreduce_add_rmsnorm);
}
