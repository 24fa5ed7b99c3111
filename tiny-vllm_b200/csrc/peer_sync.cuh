// Device helpers for kernels that exchange data with other GPUs of the node through peer
// memory: system-scope flag stores and loads, a bounded wait, 16-byte peer accesses and the
// fp32 summation of packed 16-bit values.  Plain loads and stores only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace b200q {

constexpr long long kSpinLimitCycles = 2000000000LL;  // about one second

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  // weak load, not cached in L1: each address is read once per call and the call's first
  // barrier orders it after the peers' writes
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_peer16(void* p, const uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// Waits until the flag holds at least `epoch` (wrap-safe).  False when the limit ran out.
__device__ __forceinline__ bool wait_flag(const unsigned int* flag, unsigned int epoch) {
  const long long t0 = clock64();
  while (static_cast<int>(ld_acquire_sys(flag) - epoch) < 0) {
    if (clock64() - t0 > kSpinLimitCycles) return false;
  }
  return true;
}

// Same bytes through a volatile (relaxed, system-scope) load: for data another GPU wrote
// into THIS GPU's memory during the running kernel.
__device__ __forceinline__ uint4 ld_volatile16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

template <bool BF16>
__device__ __forceinline__ void accumulate(float (&acc)[8], const uint4 v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f;
    if (BF16) {
      f = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u));
    } else {
      f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    }
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

template <bool BF16>
__device__ __forceinline__ uint4 pack(const float (&acc)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (BF16) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    } else {
      const __half2 h = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

}  // namespace b200q
