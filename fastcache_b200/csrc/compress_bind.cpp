// Bindings of the in-pool compression kernels (evict.cu, ccm.cu).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <vector>

#include "kernels.h"

namespace {
using torch::Tensor;

void check_pool(const Tensor& pool) {
  TORCH_CHECK(pool.is_cuda() && pool.scalar_type() == torch::kBFloat16 && pool.dim() == 6 && pool.is_contiguous() &&
                  pool.size(1) == 2, "pool must be contiguous bf16 [L, 2, blocks, Hkv, block, D]");
}
void check_i32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kInt32 && t.is_contiguous(), name, " must be int32 CUDA");
}

// scores [n_seq, L, Hkv, s_stride] fp32; mode 0: -||k|| per head, mode 1: +mean_heads ||k||
Tensor knorm_scores(const Tensor& pool, const Tensor& block_tables, const Tensor& kv_lens, int64_t max_len,
                    int64_t mode, Tensor status) {
  check_pool(pool);
  check_i32(block_tables, "block_tables");
  check_i32(kv_lens, "kv_lens");
  const int64_t n = kv_lens.numel(), L = pool.size(0), Hkv = pool.size(3);
  const int64_t stride = (max_len + 3) / 4 * 4;
  c10::cuda::CUDAGuard guard(pool.device());
  Tensor scores = torch::empty({n, L, Hkv, stride}, pool.options().dtype(torch::kFloat32));
  fc::launch_knorm_scores(pool.data_ptr(), block_tables.data_ptr<int>(), kv_lens.data_ptr<int>(),
                          scores.data_ptr<float>(), int(n), int(L), int(pool.size(2)), int(pool.size(4)), int(Hkv),
                          int(pool.size(5)), int(block_tables.size(1)), int(max_len), int(stride), int(mode),
                          reinterpret_cast<uint32_t*>(status.data_ptr<int>()), at::cuda::getCurrentCUDAStream());
  return scores;
}

// SnapKV scores [n_seq, L, Hkv, stride] from the observation-window queries qw [n_seq, L, w, Hq, D]
Tensor snapkv_scores(const Tensor& pool, const Tensor& block_tables, const Tensor& kv_lens, int64_t max_len,
                     const Tensor& qw, int64_t kernel_size, double scale, Tensor status) {
  check_pool(pool);
  check_i32(block_tables, "block_tables");
  check_i32(kv_lens, "kv_lens");
  const int64_t n = kv_lens.numel(), L = pool.size(0), Hkv = pool.size(3), D = pool.size(5);
  TORCH_CHECK(qw.is_cuda() && qw.scalar_type() == torch::kBFloat16 && qw.is_contiguous() && qw.dim() == 5 &&
                  qw.size(0) == n && qw.size(1) == L && qw.size(4) == D,
              "window queries must be contiguous bf16 [n_seq, L, w, Hq, D]");
  const int64_t w = qw.size(2), Hq = qw.size(3);
  const int64_t stride = (max_len + 3) / 4 * 4;
  c10::cuda::CUDAGuard guard(pool.device());
  Tensor votes = torch::empty({n, L, Hkv, stride}, pool.options().dtype(torch::kFloat32));
  Tensor scores = torch::empty({n, L, Hkv, stride}, pool.options().dtype(torch::kFloat32));
  fc::launch_snapkv_scores(pool.data_ptr(), qw.data_ptr(), block_tables.data_ptr<int>(), kv_lens.data_ptr<int>(),
                           votes.data_ptr<float>(), scores.data_ptr<float>(), int(n), int(L), int(pool.size(2)),
                           int(Hkv), int(Hq), int(pool.size(4)), int(D), int(block_tables.size(1)), int(stride),
                           int(w), int(kernel_size), float(scale),
                           reinterpret_cast<uint32_t*>(status.data_ptr<int>()), at::cuda::getCurrentCUDAStream());
  return scores;
}

// ExpectedAttention scores (log domain) from the window queries qw [n_seq, L, w, Hq, D]
Tensor expected_attention_scores(const Tensor& pool, const Tensor& block_tables, const Tensor& kv_lens,
                                 int64_t max_len, const Tensor& qw, int64_t n_sink, Tensor status) {
  check_pool(pool);
  check_i32(block_tables, "block_tables");
  check_i32(kv_lens, "kv_lens");
  const int64_t n = kv_lens.numel(), L = pool.size(0), Hkv = pool.size(3), D = pool.size(5);
  TORCH_CHECK(qw.is_cuda() && qw.scalar_type() == torch::kBFloat16 && qw.is_contiguous() && qw.dim() == 5 &&
                  qw.size(0) == n && qw.size(1) == L && qw.size(4) == D,
              "window queries must be contiguous bf16 [n_seq, L, w, Hq, D]");
  const int64_t stride = (max_len + 3) / 4 * 4;
  c10::cuda::CUDAGuard guard(pool.device());
  auto f32 = pool.options().dtype(torch::kFloat32);
  Tensor stats = torch::empty({n, L, Hkv, D + D * D}, f32);
  Tensor scores = torch::empty({n, L, Hkv, stride}, f32);
  Tensor sig16;                                      // Sigma as hi + lo bf16 for the tensor-core kernel
  if (D == 128 && fc::ea_tensor_cores()) sig16 = torch::empty({n, L, Hkv, 2, D, D}, pool.options());
  fc::launch_expected_attention_scores(pool.data_ptr(), qw.data_ptr(), block_tables.data_ptr<int>(),
                                       kv_lens.data_ptr<int>(), stats.data_ptr<float>(), scores.data_ptr<float>(),
                                       int(n), int(L), int(pool.size(2)), int(Hkv), int(qw.size(3)), int(pool.size(4)),
                                       int(D), int(block_tables.size(1)), int(stride), int(qw.size(2)), int(n_sink),
                                       reinterpret_cast<uint32_t*>(status.data_ptr<int>()),
                                       at::cuda::getCurrentCUDAStream(), sig16.defined() ? sig16.data_ptr() : nullptr);
  return scores;
}

// StreamingLLM scores: position, sinks always kept
Tensor position_scores(const Tensor& pool, const Tensor& kv_lens, int64_t max_len, int64_t n_sink) {
  check_pool(pool);
  check_i32(kv_lens, "kv_lens");
  const int64_t n = kv_lens.numel(), L = pool.size(0), Hkv = pool.size(3);
  const int64_t stride = (max_len + 3) / 4 * 4;
  c10::cuda::CUDAGuard guard(pool.device());
  Tensor scores = torch::empty({n, L, Hkv, stride}, pool.options().dtype(torch::kFloat32));
  fc::launch_position_scores(scores.data_ptr<float>(), kv_lens.data_ptr<int>(), int(n), int(L * Hkv), int(stride),
                             int(n_sink), at::cuda::getCurrentCUDAStream());
  return scores;
}

void select_compact(Tensor pool, const Tensor& scores, const Tensor& block_tables, const Tensor& kv_lens,
                    const Tensor& n_kepts, Tensor status) {
  check_pool(pool);
  check_i32(block_tables, "block_tables");
  check_i32(kv_lens, "kv_lens");
  check_i32(n_kepts, "n_kepts");
  TORCH_CHECK(scores.is_cuda() && scores.scalar_type() == torch::kFloat32 && scores.dim() == 4 &&
                  scores.is_contiguous(), "scores must be contiguous fp32 [n_seq, L, Hkv, stride]");
  TORCH_CHECK(scores.size(0) == kv_lens.numel() && scores.size(1) == pool.size(0) && scores.size(2) == pool.size(3),
              "scores do not match the pool / batch");
  c10::cuda::CUDAGuard guard(pool.device());
  fc::launch_select_compact(pool.data_ptr(), scores.data_ptr<float>(), block_tables.data_ptr<int>(),
                            kv_lens.data_ptr<int>(), n_kepts.data_ptr<int>(), int(kv_lens.numel()),
                            int(pool.size(0)), int(pool.size(2)), int(pool.size(4)), int(pool.size(3)),
                            int(pool.size(5)), int(block_tables.size(1)), int(scores.size(3)),
                            reinterpret_cast<uint32_t*>(status.data_ptr<int>()), at::cuda::getCurrentCUDAStream());
}
// In-place CCM merge of `kv_lens.numel()` requests for pool layers [layer_start, layer_end).
// Weights are the packed [Lw, 4, ...] tensors; weight_layer_start is the index of pool layer
// `layer_start` inside them.
void ccm_compress(Tensor pool, const Tensor& block_tables, const Tensor& kv_lens, const Tensor& image_lens,
                  const Tensor& w1, const Tensor& b1, const Tensor& w2, const Tensor& b2, const Tensor& w3,
                  const Tensor& b3, int64_t layer_start, int64_t layer_end, int64_t weight_layer_start,
                  int64_t factor, int64_t min_seq_len, bool single_segment, Tensor status, int64_t heads_per_cta,
                  const c10::optional<Tensor>& dst_block_tables) {
  check_pool(pool);
  check_i32(block_tables, "block_tables");
  check_i32(kv_lens, "kv_lens");
  check_i32(image_lens, "image_lens");
  const int64_t D = pool.size(5);
  for (const Tensor* t : {&w1, &b1, &w2, &b2, &w3, &b3})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kBFloat16 && t->is_contiguous(),
                "compressor weights must be contiguous bf16 CUDA tensors");
  TORCH_CHECK(w1.dim() == 4 && w1.size(1) == 4 && w1.size(2) == D && w1.size(3) == D * factor,
              "w1 must be [L, 4, D, D * factor]");
  TORCH_CHECK(w2.sizes() == w3.sizes() && w2.size(2) == D && w2.size(3) == D, "w2 / w3 must be [L, 4, D, D]");
  TORCH_CHECK(layer_start >= 0 && layer_end <= pool.size(0) && weight_layer_start >= 0 &&
                  weight_layer_start + (layer_end - layer_start) <= w1.size(0), "layer range out of bounds");
  const int* dst = nullptr;
  if (dst_block_tables.has_value() && dst_block_tables->defined()) {
    check_i32(*dst_block_tables, "dst_block_tables");
    TORCH_CHECK(dst_block_tables->sizes() == block_tables.sizes(), "dst_block_tables must have the shape of block_tables");
    dst = dst_block_tables->data_ptr<int>();
  }
  c10::cuda::CUDAGuard guard(pool.device());
  fc::launch_ccm_fused(pool.data_ptr(), block_tables.data_ptr<int>(), kv_lens.data_ptr<int>(),
                       image_lens.data_ptr<int>(), w1.data_ptr(), w2.data_ptr(), w3.data_ptr(), b1.data_ptr(),
                       b2.data_ptr(), b3.data_ptr(), int(kv_lens.numel()), int(w1.size(0)), int(layer_start),
                       int(layer_end), int(weight_layer_start), int(pool.size(2)), int(pool.size(3)),
                       int(pool.size(4)), int(D), int(block_tables.size(1)), int(factor), int(min_seq_len),
                       single_segment ? 1 : 0, int(heads_per_cta), reinterpret_cast<uint32_t*>(status.data_ptr<int>()),
                       at::cuda::getCurrentCUDAStream(), dst);
}
// ---------------------------------------------------------------------------------------- quantisers
// x: contiguous bf16 [..., D]; group size g divides D.  Returns (codes uint8, scale fp32 [..., D / g, 1], zero or
// an empty tensor).  Codes: [..., D] bytes (INT8 two's complement, FP8 bit patterns) or [..., D / 2] for the 4-bit modes.
std::vector<Tensor> quantize_rows(const Tensor& x, int64_t mode, int64_t g) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.dim() >= 1,
              "x must be a contiguous bf16 CUDA tensor");
  const int64_t D = x.size(-1);
  TORCH_CHECK(g > 0 && D % g == 0 && g % 8 == 0 && g <= 1024, "group size must divide the last dim, be a multiple of 8 and <= 1024");
  const int64_t groups = x.numel() / g;
  const bool four = mode == fc::QUANT_INT4 || mode == fc::QUANT_NF4;
  c10::cuda::CUDAGuard guard(x.device());
  auto qshape = x.sizes().vec();
  if (four) qshape.back() = D / 2;
  auto sshape = x.sizes().vec();
  sshape.back() = D / g;
  sshape.push_back(1);
  Tensor q = torch::empty(qshape, x.options().dtype(torch::kUInt8));
  Tensor scale = torch::empty(sshape, x.options().dtype(torch::kFloat32));
  Tensor zero = mode == fc::QUANT_INT8_ASYM ? torch::empty(sshape, x.options().dtype(torch::kFloat32))
                                            : torch::empty({0}, x.options().dtype(torch::kFloat32));
  fc::launch_quantize(x.data_ptr(), q.data_ptr(), scale.data_ptr<float>(),
                      zero.numel() ? zero.data_ptr<float>() : nullptr, nullptr, groups, int(g), int(mode),
                      at::cuda::getCurrentCUDAStream());
  return {q, scale, zero};
}

Tensor dequantize_rows(const Tensor& q, const Tensor& scale, const c10::optional<Tensor>& zero, int64_t mode, int64_t g) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == torch::kUInt8 && q.is_contiguous(), "codes must be contiguous uint8");
  TORCH_CHECK(scale.is_cuda() && scale.scalar_type() == torch::kFloat32 && scale.is_contiguous(), "scale must be fp32");
  const bool four = mode == fc::QUANT_INT4 || mode == fc::QUANT_NF4;
  auto shape = q.sizes().vec();
  if (four) shape.back() *= 2;
  const int64_t D = shape.back();
  TORCH_CHECK(g > 0 && D % g == 0 && g % 8 == 0, "bad group size");
  const int64_t groups = q.numel() * (four ? 2 : 1) / g;
  TORCH_CHECK(scale.numel() == groups, "one scale per group");
  const float* zp = nullptr;
  if (mode == fc::QUANT_INT8_ASYM) {
    TORCH_CHECK(zero.has_value() && zero->numel() == groups && zero->scalar_type() == torch::kFloat32, "zero points missing");
    zp = zero->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(q.device());
  Tensor y = torch::empty(shape, q.options().dtype(torch::kBFloat16));
  fc::launch_dequantize(q.data_ptr(), scale.data_ptr<float>(), zp, y.data_ptr(), groups, int(g), int(mode),
                        at::cuda::getCurrentCUDAStream());
  return y;
}

// decode(encode(x)) in one pass, no codes written
Tensor fake_quantize_rows(const Tensor& x, int64_t mode, int64_t g) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous(), "x must be a contiguous bf16 CUDA tensor");
  const int64_t D = x.size(-1);
  TORCH_CHECK(g > 0 && D % g == 0 && g % 8 == 0 && g <= 1024, "group size must divide the last dim, be a multiple of 8 and <= 1024");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  fc::launch_quantize(x.data_ptr(), nullptr, nullptr, nullptr, y.data_ptr(), x.numel() / g, int(g), int(mode),
                      at::cuda::getCurrentCUDAStream());
  return y;
}
}  // namespace

void register_compress(pybind11::module_& m) {
  m.def("quantize_rows", &quantize_rows);
  m.def("dequantize_rows", &dequantize_rows, pybind11::arg("q"), pybind11::arg("scale"), pybind11::arg("zero") = pybind11::none(),
        pybind11::arg("mode") = 0, pybind11::arg("g") = 128);
  m.def("fake_quantize_rows", &fake_quantize_rows);
  m.def("knorm_scores", &knorm_scores);
  m.def("select_compact", &select_compact);
  m.def("snapkv_scores", &snapkv_scores);
  m.def("expected_attention_scores", &expected_attention_scores);
  m.def("position_scores", &position_scores);
  m.def("set_snapkv_tensor_cores", &fc::set_snapkv_tensor_cores, "SnapKV votes on tcgen05 (head_dim 128)");
  m.def("snapkv_tensor_cores", &fc::snapkv_tensor_cores);
  m.def("set_ea_tensor_cores", &fc::set_ea_tensor_cores, "ExpectedAttention scores on tcgen05 (head_dim 128)");
  m.def("ea_tensor_cores", &fc::ea_tensor_cores);
  namespace py = pybind11;
  m.def("ccm_compress", &ccm_compress, py::arg("pool"), py::arg("block_tables"), py::arg("kv_lens"),
        py::arg("image_lens"), py::arg("w1"), py::arg("b1"), py::arg("w2"), py::arg("b2"), py::arg("w3"),
        py::arg("b3"), py::arg("layer_start"), py::arg("layer_end"), py::arg("weight_layer_start"),
        py::arg("factor"), py::arg("min_seq_len"), py::arg("single_segment"), py::arg("status"),
        py::arg("heads_per_cta") = 1, py::arg("dst_block_tables") = py::none());
}
