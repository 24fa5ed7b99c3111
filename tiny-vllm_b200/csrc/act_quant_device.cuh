// Device pieces shared by the activation quantiser and its fused producers (RMSNorm, SiLU-mul,
// the tensor-parallel reduce + RMSNorm): 16-bit unpacking, the packed absolute maximum, the
// bit-exact int8 conversion of eight values at a time, row-group reductions and the common
// "quantise the row held in registers" tail.
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
// int8 code; r = u - 1.5 * 2^23 is that integer exactly (its negative is formed by one fused
// multiply-add, -1 * u + 1.5 * 2^23, exact too) and fma(v, 1/scale, -r) the distance to it.  |p| cannot exceed 127 (1 + 2^-22) because scale >= absmax / 127, so no clamp is
// needed.  Packed fp32x2 instructions round each half like the scalar ones.
template <typename T>
__device__ __forceinline__ uint2 quant8(const uint4 raw, float scale, float inv_scale) {
  const float2 inv2 = make_float2(inv_scale, inv_scale);
  const float2 magic = make_float2(12582912.0f, 12582912.0f);      // 1.5 * 2^23
  const float2 minus_one = make_float2(-1.0f, -1.0f);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t ub[8];
  float worst = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = unpack2<T>(w[i]);
    const float2 u = __ffma2_rn(v, inv2, magic);
    const float2 nr = __ffma2_rn(u, minus_one, magic);  // -(u - magic), exact: minus the rounded integer
    const float2 d = __ffma2_rn(v, inv2, nr);
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

// ---- pieces of the kernels that form a row in registers (RMSNorm, SiLU-mul, the
// tensor-parallel reduce + RMSNorm) and quantise it there
template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Two 16-bit values times two 16-bit weights, rounded once to 16 bit (what a 16-bit tensor
// multiply does).
template <typename T>
__device__ __forceinline__ uint32_t mul2_16(uint32_t a, uint32_t w);
template <>
__device__ __forceinline__ uint32_t mul2_16<__nv_bfloat16>(uint32_t a, uint32_t w) {
  const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a),
                                   *reinterpret_cast<const __nv_bfloat162*>(&w));
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <>
__device__ __forceinline__ uint32_t mul2_16<__half>(uint32_t a, uint32_t w) {
  const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&w));
  return *reinterpret_cast<const uint32_t*>(&r);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

// Reduction over the G threads of a row group (warps of a group are neighbours in the CTA).
template <int G, bool IS_MAX>
__device__ __forceinline__ float group_reduce(float v, float* red, int g) {
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  if (G > 32) {
    constexpr int kWarpsPerRow = G / 32;
    __syncthreads();  // red may still be read from the previous reduction
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = red[g * kWarpsPerRow];
#pragma unroll
    for (int i = 1; i < kWarpsPerRow; ++i)
      m = IS_MAX ? fmaxf(m, red[g * kWarpsPerRow + i]) : m + red[g * kWarpsPerRow + i];
    v = m;
  }
  return v;
}

// Common tail: y (CHUNKS chunks of 8 values per thread) -> optional store, absmax, int8 codes.
template <typename T, int G, int CHUNKS>
__device__ __forceinline__ void quantise_row(const uint4 (&y)[CHUNKS], bool active, int row, int t,
                                             int g, int nchunk, int K, T* __restrict__ y_out,
                                             int8_t* __restrict__ xq, float* __restrict__ a_scales,
                                             float* red) {
  AbsMax2<T> running;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    running.add(y[c].x);
    running.add(y[c].y);
    running.add(y[c].z);
    running.add(y[c].w);
  }
  const float amax = group_reduce<G, true>(running.value(), red, g);
  if (!active) return;
  const float scale = fmaxf(__fdiv_rn(amax, 127.0f), 1e-8f);
  const float inv_scale = __frcp_rn(scale);
  if (t == 0) a_scales[row] = scale;
  uint2* dst = reinterpret_cast<uint2*>(xq + static_cast<size_t>(row) * K);
  uint4* ydst = y_out != nullptr ? reinterpret_cast<uint4*>(y_out + static_cast<size_t>(row) * K) : nullptr;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int idx = c * G + t;
    if (idx < nchunk) {
      dst[idx] = quant8<T>(y[c], scale, inv_scale);
      if (ydst != nullptr) ydst[idx] = y[c];
    }
  }
}


}  // namespace
}  // namespace b200q
