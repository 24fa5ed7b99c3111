// Device helpers for kernels that exchange data with other GPUs of the node through peer
// memory: system-scope flag stores and loads, a bounded wait, 16-byte peer accesses and the
// fp32 summation of packed 16-bit values.  Plain loads and stores only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace b200q {

// Default limit of one wait on a peer, in SM cycles (about one second).  The launchers pass
// the limit to the kernels as a parameter, so that a test can shorten it to milliseconds.
constexpr long long kSpinLimitCycles = 2000000000LL;

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
__device__ __forceinline__ bool wait_flag(const unsigned int* flag, unsigned int epoch,
                                          long long limit_cycles) {
  const long long t0 = clock64();
  while (static_cast<int>(ld_acquire_sys(flag) - epoch) < 0) {
    if (clock64() - t0 > limit_cycles) return false;
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


// ---- tagged words: the exchange format of the one-trip kernels (fused decode GEMM +
// all-reduce, small all-reduce).  A value pair travels as an aligned 8-byte word {data,
// call number}; such a store arrives whole, so a word whose tag equals the current call
// number is valid data and no fence or separate flag is needed.
constexpr int kCtlEpoch = 0;    // control word: calls completed by this rank
constexpr int kCtlCounter = 1;  // control word: CTAs of the running call that are done

__device__ __forceinline__ void st_word8(void* p, uint32_t data, uint32_t tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(data), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ld_word8(const void* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
// Polls a tagged word until it carries `epoch`; false when the limit ran out.
__device__ __forceinline__ bool wait_word8(const void* p, uint32_t epoch, uint32_t* data,
                                           long long limit_cycles) {
  uint2 v = ld_word8(p);
  if (v.y != epoch) {
    const long long t0 = clock64();
    do {
      v = ld_word8(p);
    } while (v.y != epoch && clock64() - t0 < limit_cycles);
  }
  *data = v.x;
  return v.y == epoch;
}
// The call number of the launch that is starting (0 is never used as a tag).
__device__ __forceinline__ unsigned int next_epoch(const unsigned int* ctl) {
  unsigned int e = *reinterpret_cast<const volatile unsigned int*>(ctl + kCtlEpoch) + 1u;
  return e == 0u ? 1u : e;
}
// Called by one thread per CTA at the end: the last CTA publishes the finished call number.
__device__ __forceinline__ void finish_call(unsigned int* ctl, unsigned int epoch) {
  if (atomicAdd(ctl + kCtlCounter, 1u) == gridDim.x - 1) {
    ctl[kCtlCounter] = 0u;
    *reinterpret_cast<volatile unsigned int*>(ctl + kCtlEpoch) = epoch;
  }
}

}  // namespace b200q
