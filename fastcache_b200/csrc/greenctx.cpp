// Green-context runtime: split the device's SMs into two disjoint groups and hand
// back one stream per group.
//
// The reference obtains this from an external wheel
// (sgl_kernel.create_greenctx_stream_by_value, called in
// "kv-cache pipeline"/nanovllm/utils/streams.py:50-86) and needs a preload shim to
// import it; here it is part of the extension.  Driver entry points are resolved at
// run time so the module loads on machines without a driver (CPU build checks).
#include <cuda.h>
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

namespace py = pybind11;

namespace {

// `version`: the CUDA release that introduced the entry point (green contexts: 12.4;
// cuGreenCtxStreamCreate: 12.5).  Asking for a symbol at an older version than its first
// one reports "not found" even on a newer driver.
template <typename Fn>
Fn resolve(const char* name, unsigned version = 12040) {
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPointByVersion(name, &ptr, version, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || ptr == nullptr)
    throw std::runtime_error(std::string("driver entry point not available: ") + name);
  return reinterpret_cast<Fn>(ptr);
}

void check(CUresult r, const char* what) {
  if (r != CUDA_SUCCESS) throw std::runtime_error(std::string(what) + " failed with CUresult " + std::to_string(int(r)));
}

using DeviceGetFn = CUresult (*)(CUdevice*, int);
using GetDevResourceFn = CUresult (*)(CUdevice, CUdevResource*, CUdevResourceType);
using SplitFn = CUresult (*)(CUdevResource*, unsigned int*, const CUdevResource*, CUdevResource*, unsigned int,
                             unsigned int);
using GenDescFn = CUresult (*)(CUdevResourceDesc*, CUdevResource*, unsigned int);
using GreenCreateFn = CUresult (*)(CUgreenCtx*, CUdevResourceDesc, CUdevice, unsigned int);
using GreenStreamFn = CUresult (*)(CUstream*, CUgreenCtx, unsigned int, int);
using GreenDestroyFn = CUresult (*)(CUgreenCtx);
using StreamDestroyFn = CUresult (*)(CUstream);

struct Partition {
  CUgreenCtx ctx[2] = {nullptr, nullptr};
  CUstream stream[2] = {nullptr, nullptr};
  int sms[2] = {0, 0};
};
std::vector<Partition> g_live;
std::mutex g_mu;

// Returns {main_stream, compress_stream, main_sms, compress_sms, total_sms}.
// `compress_sms` is a request; the driver rounds it to its SM-group granularity.
py::dict create_partition(int device, int compress_sms, int main_priority, int compress_priority) {
  cudaSetDevice(device);
  cudaFree(nullptr);   // make sure the primary context exists
  auto deviceGet = resolve<DeviceGetFn>("cuDeviceGet");
  auto getRes = resolve<GetDevResourceFn>("cuDeviceGetDevResource");
  auto split = resolve<SplitFn>("cuDevSmResourceSplitByCount");
  auto genDesc = resolve<GenDescFn>("cuDevResourceGenerateDesc");
  auto greenCreate = resolve<GreenCreateFn>("cuGreenCtxCreate");
  auto greenStream = resolve<GreenStreamFn>("cuGreenCtxStreamCreate", 12050);

  CUdevice dev;
  check(deviceGet(&dev, device), "cuDeviceGet");
  CUdevResource all;
  check(getRes(dev, &all, CU_DEV_RESOURCE_TYPE_SM), "cuDeviceGetDevResource");
  const int total = int(all.sm.smCount);
  if (compress_sms <= 0 || compress_sms >= total) throw std::runtime_error("compress_sms must be in (0, total SMs)");

  // carve the main group by count; what is left over is the compression group
  const unsigned want_main = unsigned(total - compress_sms);
  CUdevResource main_res, rest;
  unsigned groups = 1;
  check(split(&main_res, &groups, &all, &rest, 0, want_main), "cuDevSmResourceSplitByCount");
  if (groups < 1 || rest.sm.smCount == 0) throw std::runtime_error("SM split left no SMs for the second group");

  Partition p;
  CUdevResource parts[2] = {main_res, rest};
  const int prio[2] = {main_priority, compress_priority};
  for (int i = 0; i < 2; ++i) {
    CUdevResourceDesc desc;
    check(genDesc(&desc, &parts[i], 1), "cuDevResourceGenerateDesc");
    check(greenCreate(&p.ctx[i], desc, dev, CU_GREEN_CTX_DEFAULT_STREAM), "cuGreenCtxCreate");
    check(greenStream(&p.stream[i], p.ctx[i], CU_STREAM_NON_BLOCKING, prio[i]), "cuGreenCtxStreamCreate");
    p.sms[i] = int(parts[i].sm.smCount);
  }
  {
    std::lock_guard<std::mutex> lk(g_mu);
    g_live.push_back(p);
  }
  py::dict d;
  d["main_stream"] = reinterpret_cast<uint64_t>(p.stream[0]);
  d["compress_stream"] = reinterpret_cast<uint64_t>(p.stream[1]);
  d["main_sms"] = p.sms[0];
  d["compress_sms"] = p.sms[1];
  d["total_sms"] = total;
  return d;
}

// Extra stream on an existing partition's compression group (round-robin compression streams).
uint64_t extra_compress_stream(uint64_t compress_stream, int priority) {
  auto greenStream = resolve<GreenStreamFn>("cuGreenCtxStreamCreate", 12050);
  std::lock_guard<std::mutex> lk(g_mu);
  for (auto& p : g_live) {
    if (reinterpret_cast<uint64_t>(p.stream[1]) == compress_stream) {
      CUstream s;
      check(greenStream(&s, p.ctx[1], CU_STREAM_NON_BLOCKING, priority), "cuGreenCtxStreamCreate");
      return reinterpret_cast<uint64_t>(s);
    }
  }
  throw std::runtime_error("unknown green-context partition");
}

int sm_count(int device) {
  int n = 0;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
  return n;
}

// Destroys every partition created by this process.  Streams must be idle.
void destroy_all() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_live.empty()) return;
  auto greenDestroy = resolve<GreenDestroyFn>("cuGreenCtxDestroy");
  auto streamDestroy = resolve<StreamDestroyFn>("cuStreamDestroy");
  for (auto& p : g_live) {
    for (int i = 0; i < 2; ++i) {
      if (p.stream[i]) streamDestroy(p.stream[i]);
      if (p.ctx[i]) greenDestroy(p.ctx[i]);
    }
  }
  g_live.clear();
}

}  // namespace

void register_greenctx(py::module_& m) {
  m.def("greenctx_create", &create_partition, py::arg("device"), py::arg("compress_sms"),
        py::arg("main_priority") = 0, py::arg("compress_priority") = 0);
  m.def("greenctx_extra_stream", &extra_compress_stream);
  m.def("greenctx_destroy_all", &destroy_all);
  m.def("sm_count", &sm_count);
}
