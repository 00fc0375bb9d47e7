// Release/acquire counters in peer-visible memory: the building blocks of every
// kernel that talks to another GPU.  Counters only grow, waits are ">=" in
// wrap-around arithmetic and every wait is bounded: on time-out the caller gets
// `false` and the status word holds kStatusPeerWaitTimeout; nothing traps.
#pragma once
#include "../common/ptx.cuh"

namespace nfb {

constexpr uint32_t kPeerPollLimit = 1u << 22;

__device__ __forceinline__ uint32_t ld_acquire_sys(const unsigned int* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned int* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// 16-byte load that is never served from a stale L1 line (polling of data another GPU writes).
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Same counter when producer and consumer are known to be on one GPU: device scope is enough and far cheaper when
// thousands of CTAs signal one word.
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Wait until *flag - target >= 0 in wrap-around arithmetic.  Returns false on time-out, and at once (after one
// look at the counter) when the status word already holds a failure: after the first wait that ran out, the
// kernels that follow it in the stream would otherwise each spend their own full limit.
__device__ __forceinline__ bool wait_counter(const unsigned int* flag, uint32_t target, int* status) {
  for (uint32_t i = 0; i < kPeerPollLimit; ++i) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - target) >= 0) return true;
    if ((i & 1023u) == 0 && status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return false;
    __nanosleep(i < 64 ? 20 : 200);
  }
  report_status(status, kStatusPeerWaitTimeout);
  return false;
}

}  // namespace nfb
