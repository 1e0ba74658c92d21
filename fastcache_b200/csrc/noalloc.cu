// Allocation-free variant of split-KV decode attention: see noalloc.h for the contract.
#include "noalloc.h"

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <exception>
#include <mutex>

#include "kernels.h"

namespace {

// Scratch of the split-KV path, owned by the library instead of the caller.
static __device__ __align__(256) float g_part_o[FC_NOALLOC_MAX_PART_FLOATS];
static __device__ __align__(256) float g_part_lse[FC_NOALLOC_MAX_LSE_FLOATS];

constexpr int MAX_DEVICES = 64;
struct DeviceScratch {
  float* part_o = nullptr;
  float* part_lse = nullptr;
};
DeviceScratch g_scratch[MAX_DEVICES];
std::mutex g_mu;

void set_err(char* err, size_t n, const char* msg) {
  if (err != nullptr && n > 0) snprintf(err, n, "%s", msg);
}

// In host code the array names are host-side handles, not device addresses; the device
// addresses come from cudaGetSymbolAddress, once per device, with that device current.
int resolve(int dev, DeviceScratch* out, char* err, size_t err_len) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_scratch[dev].part_o == nullptr) {
    void* po = nullptr;
    void* pl = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&po, g_part_o);
    if (e != cudaSuccess) {
      set_err(err, err_len, cudaGetErrorString(e));
      return FC_NOALLOC_CUDA_ERROR;
    }
    e = cudaGetSymbolAddress(&pl, g_part_lse);
    if (e != cudaSuccess) {
      set_err(err, err_len, cudaGetErrorString(e));
      return FC_NOALLOC_CUDA_ERROR;
    }
    g_scratch[dev].part_o = static_cast<float*>(po);
    g_scratch[dev].part_lse = static_cast<float*>(pl);
  }
  *out = g_scratch[dev];
  return FC_NOALLOC_OK;
}

}  // namespace

extern "C" int fc_decode_attention_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                           const int* block_tables, const int* context_lens, void* out, int B,
                                           int Hq, int Hkv, int D, int block_size, int max_blocks, int num_blocks,
                                           int splits, float scale, unsigned int* status, void* stream, char* err,
                                           size_t err_len) {
  if (q == nullptr || k_cache == nullptr || v_cache == nullptr || block_tables == nullptr ||
      context_lens == nullptr || out == nullptr) {
    set_err(err, err_len, "null pointer argument");
    return FC_NOALLOC_BAD_ARGUMENT;
  }
  if (B < 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > 16 || (D != 64 && D != 128) || splits < 1 ||
      splits > fc::DECODE_MAX_SPLITS || block_size < 8 || block_size % 8 != 0 || max_blocks <= 0 ||
      num_blocks <= 0) {
    set_err(err, err_len,
            "unsupported shape: need Hq % Hkv == 0, Hq / Hkv <= 16, D in {64, 128}, 1 <= splits <= 32, "
            "block_size a multiple of 8");
    return FC_NOALLOC_BAD_ARGUMENT;
  }
  const unsigned long long part = (unsigned long long)B * Hq * splits * D;
  const unsigned long long lse = (unsigned long long)B * Hq * splits;
  if (part > FC_NOALLOC_MAX_PART_FLOATS || lse > FC_NOALLOC_MAX_LSE_FLOATS) {
    char msg[200];
    snprintf(msg, sizeof(msg),
             "request needs %llu partial floats and %llu lse floats; the static scratch holds %u and %u "
             "(reduce B, Hq or splits)",
             part, lse, FC_NOALLOC_MAX_PART_FLOATS, FC_NOALLOC_MAX_LSE_FLOATS);
    set_err(err, err_len, msg);
    return FC_NOALLOC_TOO_LARGE;
  }
  if (B == 0) return FC_NOALLOC_OK;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    set_err(err, err_len, e != cudaSuccess ? cudaGetErrorString(e) : "device ordinal out of range");
    return FC_NOALLOC_CUDA_ERROR;
  }
  DeviceScratch s;
  const int rc = resolve(dev, &s, err, err_len);
  if (rc != FC_NOALLOC_OK) return rc;
  try {
    fc::launch_decode_attention(q, k_cache, v_cache, block_tables, context_lens, out, s.part_o, s.part_lse, B, Hq,
                                Hkv, D, block_size, max_blocks, num_blocks, splits, scale, status,
                                static_cast<cudaStream_t>(stream));
  } catch (const std::exception& ex) {
    set_err(err, err_len, ex.what());
    return FC_NOALLOC_CUDA_ERROR;
  }
  return FC_NOALLOC_OK;
}
