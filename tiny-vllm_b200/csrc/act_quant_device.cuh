// Device pieces shared by the activation quantiser and its fused producers (RMSNorm, SiLU-mul):
// 16-bit unpacking, the packed absolute maximum, and the bit-exact int8 conversion of
// eight values at a time.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200q {
namespace {

template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t u);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) {
  // bf16 -> fp32 is a 16-bit shift
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t u) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}

// Running absolute maximum of a row, kept in the 16-bit domain: two elements per instruction.
// |x| of a 16-bit float compares like the float itself, so the packed maximum of the packed
// absolute values is exact; it is widened to fp32 once per thread.  (NaN elements are skipped,
// as fmaxf would.)
template <typename T>
struct AbsMax2;
template <>
struct AbsMax2<__nv_bfloat16> {
  __nv_bfloat162 m;
  __device__ __forceinline__ AbsMax2() : m(__floats2bfloat162_rn(0.f, 0.f)) {}
  __device__ __forceinline__ void add(uint32_t u) {
    m = __hmax2(m, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&u)));
  }
  __device__ __forceinline__ float value() const {
    return fmaxf(__low2float(m), __high2float(m));
  }
};
template <>
struct AbsMax2<__half> {
  __half2 m;
  __device__ __forceinline__ AbsMax2() : m(__floats2half2_rn(0.f, 0.f)) {}
  __device__ __forceinline__ void add(uint32_t u) {
    m = __hmax2(m, __habs2(*reinterpret_cast<const __half2*>(&u)));
  }
  __device__ __forceinline__ float value() const {
    return fmaxf(__low2float(m), __high2float(m));
  }
};

// Exact path for one element: clamp(rint(v / scale), -127, 127) as a byte (IEEE division).
__device__ __forceinline__ uint32_t quant1_exact(float v, float scale) {
  int q = __float2int_rn(__fdiv_rn(v, scale));  // round half to even
  q = max(-127, min(127, q));
  return static_cast<uint32_t>(q) & 0xFFu;
}

template <typename T>
__device__ __noinline__ uint2 quant8_exact(const uint4 raw, float scale) {
  const float2 a = unpack2<T>(raw.x), b = unpack2<T>(raw.y), c = unpack2<T>(raw.z),
               d = unpack2<T>(raw.w);
  uint2 o;
  o.x = quant1_exact(a.x, scale) | (quant1_exact(a.y, scale) << 8) |
        (quant1_exact(b.x, scale) << 16) | (quant1_exact(b.y, scale) << 24);
  o.y = quant1_exact(c.x, scale) | (quant1_exact(c.y, scale) << 8) |
        (quant1_exact(d.x, scale) << 16) | (quant1_exact(d.y, scale) << 24);
  return o;
}

// Eight elements -> eight int8 codes, bit-identical to the IEEE division.
// Fast path: the exact product p = v * (1/scale) is within 1.3e-5 of the rounded quotient
// fl(v / scale) (|p| <= 127; one rounding in the reciprocal, one in the quotient), hence
// rint(p) can differ from rint(fl(v / scale)) only when p lies that close to a rounding tie
// k + 0.5.  A chunk that has such an element (|p - rint(p)| > 0.4999, about one chunk in
// 600 for random data) is redone with exact divisions.  Rounding uses the 1.5 * 2^23
// trick: u = fma(v, 1/scale, 1.5 * 2^23) rounds p half-to-even to an integer and leaves
// that integer in the low mantissa bits (two's complement), i.e. the low byte of u is the
// int8 code; r = u - 1.5 * 2^23 is that integer exactly and fma(v, 1/scale, -r) the distance
// to it.  |p| cannot exceed 127 (1 + 2^-22) because scale >= absmax / 127, so no clamp is
// needed.  Packed fp32x2 instructions round each half like the scalar ones.
template <typename T>
__device__ __forceinline__ uint2 quant8(const uint4 raw, float scale, float inv_scale) {
  const float2 inv2 = make_float2(inv_scale, inv_scale);
  const float2 magic = make_float2(12582912.0f, 12582912.0f);      // 1.5 * 2^23
  const float2 neg_magic = make_float2(-12582912.0f, -12582912.0f);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t ub[8];
  float worst = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = unpack2<T>(w[i]);
    const float2 u = __ffma2_rn(v, inv2, magic);
    const float2 r = __fadd2_rn(u, neg_magic);
    const float2 d = __ffma2_rn(v, inv2, make_float2(-r.x, -r.y));
    worst = fmaxf(worst, fmaxf(fabsf(d.x), fabsf(d.y)));
    ub[2 * i] = __float_as_uint(u.x);
    ub[2 * i + 1] = __float_as_uint(u.y);
  }
  if (!(worst <= 0.4999f)) return quant8_exact<T>(raw, scale);  // also taken for NaN
  uint2 o;
  o.x = __byte_perm(__byte_perm(ub[0], ub[1], 0x0040), __byte_perm(ub[2], ub[3], 0x0040), 0x5410);
  o.y = __byte_perm(__byte_perm(ub[4], ub[5], 0x0040), __byte_perm(ub[6], ub[7], 0x0040), 0x5410);
  return o;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

}  // namespace
}  // namespace b200q
