// Device helpers shared by the kernels that talk to other GPUs (comm.cu, gemm_skinny.cu): system-scope
// release / acquire accesses, 16-byte peer loads, the NVSwitch multimem reduction and packing helpers.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include "comm.h"
#include "ptx.cuh"

namespace fc {

#ifndef FC_PEER_SPIN_LIMIT
#define FC_PEER_SPIN_LIMIT (1u << 24)      // polls before giving up; the time limit usually ends the wait first
#endif

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// sum over all ranks bound to the multicast object, 8 bf16 at a time, fp32 accumulation in the switch
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}

__device__ __forceinline__ void unpack8f(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8f(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]);
  u.y = pack_bf16(f[2], f[3]);
  u.z = pack_bf16(f[4], f[5]);
  u.w = pack_bf16(f[6], f[7]);
  return u;
}

// One thread's part of the flag exchange of CTA `slot` with the same CTA of every rank: thread `peer` posts this
// rank's arrival (`epoch`) to rank `peer` and waits for that rank's arrival here.  Everything the CTA wrote
// before the barrier that precedes this call is visible to the peer once it has seen the flag.  Returns false
// when the bounded wait ran out (the status word then holds ST_TIMEOUT_PEER).
__device__ __forceinline__ bool peer_flag_exchange(const CommPeers& peers, int slot, uint32_t epoch, int peer,
                                                   uint32_t* status) {
  st_release_sys(peers.flags[peer] + (size_t)slot * COMM_MAX_WORLD + peers.rank, epoch);
  const uint32_t* mine = peers.flags[peers.rank] + (size_t)slot * COMM_MAX_WORLD + peer;
  const uint64_t t0 = global_timer_ns();
  uint64_t limit = FC_PEER_WAIT_LIMIT_NS;
  for (uint32_t i = 0; i < FC_PEER_SPIN_LIMIT; ++i) {
    // epochs only grow; a peer that is already one exchange ahead is fine
    if (int32_t(ld_acquire_sys(mine) - epoch) >= 0) return true;
    __nanosleep(20);
    if ((i & 255u) == 255u) {
      if (i == 255u) limit = peer_wait_limit_ns(status);
      if (global_timer_ns() - t0 > limit) break;
    }
  }
  report(status, ST_TIMEOUT_PEER);
  return false;
}

}  // namespace fc
