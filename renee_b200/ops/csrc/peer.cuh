// Peer-memory signalling primitives shared by the collective kernels and the classifier GEMMs.
// Flags live in a symmetric allocation mapped on every GPU; a flag value is a monotonically increasing
// step tag, written with a system-scope release after the payload and polled with a system-scope
// acquire.  Tags are computed on the device as (*step_ptr) * mul + add, so a captured CUDA graph stays
// valid from step to step.  All waits are bounded.
#pragma once
#include "tc.cuh"

namespace rb {

constexpr int kMaxPeers = 16;
struct PeerPtrs { void* p[kMaxPeers]; };

struct StepTag {              // tag = (*step) * mul + add
  const uint32_t* step;
  uint32_t mul;
  uint32_t add;
  __device__ __forceinline__ uint32_t value() const { return (*step) * mul + add; }
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// NVLS: one load returns the sum over every GPU bound to the multicast address (reduced in the NVSwitch,
// fp32 accumulation of packed 16-bit pairs); one store lands in every GPU's copy.
template <typename T> __device__ __forceinline__ uint4 multimem_ld_reduce_v4(const void* mc_addr);
template <> __device__ __forceinline__ uint4 multimem_ld_reduce_v4<__nv_bfloat16>(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
template <> __device__ __forceinline__ uint4 multimem_ld_reduce_v4<__half>(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Bounded wait until *flag >= want (wrap-safe).  Returns false (and records status) on expiry.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t want, int* status, int detail) {
  if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
  const uint64_t t0 = tc::now_ns();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
      __nanosleep(64);
    }
    if (tc::now_ns() - t0 > tc::kWaitBudgetNs) break;
  }
  if (status != nullptr && atomicCAS(status, 0, 1000 + tc::SITE_PEER_FLAG) == 0) {
    status[1] = (int)blockIdx.x;
    status[2] = tc::SITE_PEER_FLAG;
    status[3] = detail;
  }
  return false;
}

}  // namespace rb
