// Symmetric memory for the fused tensor-parallel kernels: every rank allocates the same buffers with the CUDA
// virtual-memory API, hands the allocation to its peers as a POSIX file descriptor, maps the peers' allocations
// into its own address space (peer pointers for ld / st / red over NVLink) and, where the system supports it,
// binds all of them to one NVSwitch multicast object (the address multimem.ld_reduce / multimem.st work on).
//
// The reference has nothing of the kind (its only collectives are NCCL calls, nanovllm/utils/tp.py:112-186).
// What crosses process boundaries is done by the Python side (parallel/symm_native.py): file descriptors travel
// over Unix sockets, everything else over the torch.distributed group.  This file owns the driver calls.
//
// No tensor-memory load here is ever multicast: the multicast object is only an address range for multimem.*
// instructions issued by this package's own kernels.
#include <cuda.h>
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <unistd.h>

#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace py = pybind11;

namespace {

template <typename Fn>
Fn drv(const char* name, unsigned version = 12010) {
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPointByVersion(name, &ptr, version, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || ptr == nullptr)
    throw std::runtime_error(std::string("driver entry point not available: ") + name);
  return reinterpret_cast<Fn>(ptr);
}
void ck(CUresult r, const char* what) {
  if (r != CUDA_SUCCESS) throw std::runtime_error(std::string(what) + " failed with CUresult " + std::to_string(int(r)));
}

using MemCreateFn = CUresult (*)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
using MemGranFn = CUresult (*)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
using MemReserveFn = CUresult (*)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
using MemMapFn = CUresult (*)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
using MemAccessFn = CUresult (*)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
using MemExportFn = CUresult (*)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
using MemImportFn = CUresult (*)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
using MemUnmapFn = CUresult (*)(CUdeviceptr, size_t);
using MemFreeVaFn = CUresult (*)(CUdeviceptr, size_t);
using MemReleaseFn = CUresult (*)(CUmemGenericAllocationHandle);
using DevGetAttrFn = CUresult (*)(int*, CUdevice_attribute, CUdevice);
using McCreateFn = CUresult (*)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
using McAddDevFn = CUresult (*)(CUmemGenericAllocationHandle, CUdevice);
using McBindFn = CUresult (*)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t,
                              unsigned long long);
using McGranFn = CUresult (*)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);

struct Mapping {
  CUdeviceptr va = 0;
  size_t size = 0;
  CUmemGenericAllocationHandle handle = 0;
  bool owns_handle = false;
};
std::unordered_map<unsigned long long, Mapping> g_maps;      // by virtual address
std::mutex g_mu;

CUmemAllocationProp device_prop(int device) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

unsigned long long map_handle(CUmemGenericAllocationHandle h, size_t size, int device, bool owns) {
  CUdeviceptr va = 0;
  ck(drv<MemReserveFn>("cuMemAddressReserve")(&va, size, 0, 0, 0), "cuMemAddressReserve");
  ck(drv<MemMapFn>("cuMemMap")(va, size, 0, h, 0), "cuMemMap");
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  ck(drv<MemAccessFn>("cuMemSetAccess")(va, size, &acc, 1), "cuMemSetAccess");
  std::lock_guard<std::mutex> lk(g_mu);
  g_maps[(unsigned long long)va] = Mapping{va, size, h, owns};
  return (unsigned long long)va;
}

// Size rounded up to what both a device allocation and a multicast binding accept.
size_t symm_granularity(int device, int world) {
  cudaSetDevice(device);
  cudaFree(nullptr);
  CUmemAllocationProp prop = device_prop(device);
  size_t g = 0;
  ck(drv<MemGranFn>("cuMemGetAllocationGranularity")(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
     "cuMemGetAllocationGranularity");
  try {
    CUmulticastObjectProp mp{};
    mp.numDevices = unsigned(world);
    mp.size = g;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (drv<McGranFn>("cuMulticastGetGranularity")(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > g)
      g = mg;
  } catch (const std::exception&) {
  }
  return g;
}

// Allocate `size` bytes (a multiple of symm_granularity) on `device`, map them here, return (address, fd).
py::tuple symm_alloc(size_t size, int device) {
  cudaSetDevice(device);
  cudaFree(nullptr);
  CUmemAllocationProp prop = device_prop(device);
  CUmemGenericAllocationHandle h = 0;
  ck(drv<MemCreateFn>("cuMemCreate")(&h, size, &prop, 0), "cuMemCreate");
  int fd = -1;
  ck(drv<MemExportFn>("cuMemExportToShareableHandle")(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
     "cuMemExportToShareableHandle");
  const unsigned long long va = map_handle(h, size, device, true);
  cudaMemset(reinterpret_cast<void*>(va), 0, size);
  cudaDeviceSynchronize();
  return py::make_tuple(va, fd);
}

// Map a peer's allocation (its file descriptor arrived over a Unix socket) for access from `device`.
unsigned long long symm_import(int fd, size_t size, int device) {
  cudaSetDevice(device);
  CUmemGenericAllocationHandle h = 0;
  ck(drv<MemImportFn>("cuMemImportFromShareableHandle")(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
     "cuMemImportFromShareableHandle");
  return map_handle(h, size, device, true);
}

bool multicast_supported(int device) {
  try {
    int v = 0;
    if (drv<DevGetAttrFn>("cuDeviceGetAttribute")(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device) != CUDA_SUCCESS)
      return false;
    return v != 0;
  } catch (const std::exception&) {
    return false;
  }
}

// Rank 0: create the multicast object for `world` devices; returns (handle, fd to send to the peers).
py::tuple multicast_create(size_t size, int world) {
  CUmulticastObjectProp mp{};
  mp.numDevices = unsigned(world);
  mp.size = size;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h = 0;
  ck(drv<McCreateFn>("cuMulticastCreate")(&h, &mp), "cuMulticastCreate");
  int fd = -1;
  ck(drv<MemExportFn>("cuMemExportToShareableHandle")(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
     "cuMemExportToShareableHandle (multicast)");
  return py::make_tuple((unsigned long long)h, fd);
}
unsigned long long multicast_import(int fd) {
  CUmemGenericAllocationHandle h = 0;
  ck(drv<MemImportFn>("cuMemImportFromShareableHandle")(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
     "cuMemImportFromShareableHandle (multicast)");
  return (unsigned long long)h;
}
// Every rank, in two steps with a barrier between them (all devices must be added before any memory is bound).
void multicast_add_device(unsigned long long mc, int device) {
  ck(drv<McAddDevFn>("cuMulticastAddDevice")(CUmemGenericAllocationHandle(mc), device), "cuMulticastAddDevice");
}
// Bind this rank's allocation (the one mapped at `local_va`) and map the multicast object; returns its address.
unsigned long long multicast_bind(unsigned long long mc, unsigned long long local_va, size_t size, int device) {
  CUmemGenericAllocationHandle local = 0;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_maps.find(local_va);
    if (it == g_maps.end()) throw std::runtime_error("multicast_bind: unknown local allocation");
    local = it->second.handle;
  }
  ck(drv<McBindFn>("cuMulticastBindMem")(CUmemGenericAllocationHandle(mc), 0, local, 0, size, 0), "cuMulticastBindMem");
  return map_handle(CUmemGenericAllocationHandle(mc), size, device, false);
}

void symm_free(unsigned long long va) {
  Mapping m;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_maps.find(va);
    if (it == g_maps.end()) return;
    m = it->second;
    g_maps.erase(it);
  }
  drv<MemUnmapFn>("cuMemUnmap")(m.va, m.size);
  drv<MemFreeVaFn>("cuMemAddressFree")(m.va, m.size);
  if (m.owns_handle) drv<MemReleaseFn>("cuMemRelease")(m.handle);
}
void multicast_release(unsigned long long mc) { drv<MemReleaseFn>("cuMemRelease")(CUmemGenericAllocationHandle(mc)); }

void close_fd(int fd) {
  if (fd >= 0) ::close(fd);
}

}  // namespace

void register_symm(py::module_& m) {
  m.def("symm_granularity", &symm_granularity);
  m.def("symm_alloc", &symm_alloc);
  m.def("symm_import", &symm_import);
  m.def("symm_free", &symm_free);
  m.def("symm_close_fd", &close_fd);
  m.def("multicast_supported", &multicast_supported);
  m.def("multicast_create", &multicast_create);
  m.def("multicast_import", &multicast_import);
  m.def("multicast_add_device", &multicast_add_device);
  m.def("multicast_bind", &multicast_bind);
  m.def("multicast_release", &multicast_release);
}
