// Device-side primitives of the fused compute + collective kernels: system-scope flag signalling
// between GPUs, bounded flag waits, plain peer loads, and the `multimem` family, which acts on the
// multicast alias of a symmetric-heap buffer (one address that stands for the same offset in every
// rank's memory; the NVSwitch performs the reduction or the replication).
//
// None of these is a TMA / bulk copy: peer and multicast memory is only ever touched by ordinary
// ld / st / red / multimem instructions issued by the threads themselves.
#pragma once

#include "common.cuh"

namespace b200 {

// ---- flags ---------------------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* addr, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void red_relaxed_sys_add(uint32_t* addr, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// Spins until *addr >= target (wrap-safe) or the budget (SM cycles) runs out. One thread calls this.
__device__ __forceinline__ bool wait_flag_geq(const uint32_t* addr, uint32_t target, long long budget) {
  long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (static_cast<int32_t>(ld_acquire_sys(addr) - target) >= 0) return true;
    if ((++spins & 0x3f) == 0) {
      const long long now = clock64();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget) return false;
    }
  }
}

// ---- plain peer access ---------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* addr) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(addr)
               : "memory");
  return v;
}

// ---- multimem (addresses are multicast aliases) ---------------------------------------------------
// Sum over all ranks of eight bf16 values, accumulated in fp32 inside the switch, returned as bf16.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
// Stores of 16 / 8 / 4 bytes to every rank's copy (the f32 vector types only name the width).
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}
__device__ __forceinline__ void multimem_st_v2(void* mc_addr, const uint2& v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y))
               : "memory");
}
__device__ __forceinline__ void multimem_st_b32(void* mc_addr, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.b32 [%0], %1;" ::"l"(mc_addr), "r"(v) : "memory");
}
// Adds to a u32 counter on every rank, with release semantics (orders the caller's earlier writes).
__device__ __forceinline__ void multimem_red_release_add(uint32_t* mc_addr, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_addr), "r"(v) : "memory");
}

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

}  // namespace b200
