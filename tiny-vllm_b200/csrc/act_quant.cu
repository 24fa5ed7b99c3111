// Per-token dynamic int8 quantisation of activations, one pass over HBM.
//
//   a_scale[m] = max(absmax_k(x[m,k]) / 127, 1e-8)
//   xq[m,k]    = clamp(rint(x[m,k] / a_scale[m]), -127, 127)
//
// Same arithmetic, operation by operation, as
// nanovllm/quantization/utils.py:28-32 (fp32 absmax, IEEE division by 127, clamp_min,
// IEEE division of every element by the scale, round-half-even, clamp, cast), so the
// int8 codes and the scales are bit-identical to that function.
//
// A row is owned by a group of G threads (one warp, or one 256-thread CTA for long
// rows).  Each thread keeps its part of the row in registers (128-bit loads), the
// group reduces the absolute maximum with warp shuffles, and every thread then
// converts and stores its elements as packed 64-bit words: x is read once and xq
// written once (3 bytes of traffic per element for 16-bit inputs).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.h"
#include "ptx_sm100.cuh"

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

// G threads per row (32, 64, 128 or 256), CHUNKS 16-byte chunks per thread held in registers.
// Requires K <= G * 8 * CHUNKS.
template <typename T, int G, int CHUNKS>
__global__ void __launch_bounds__(256)
act_quant_rows_kernel(const T* __restrict__ x, int64_t ldx, int8_t* __restrict__ xq,
                      float* __restrict__ a_scales, int M, int K) {
  constexpr int kRowsPerBlock = 256 / G;
  ptx::grid_dependency_wait();     // x may be the previous kernel's output
  ptx::grid_launch_dependents();
  const int g = threadIdx.x / G;  // row group inside the block
  const int t = threadIdx.x % G;  // thread inside the group
  const int row = blockIdx.x * kRowsPerBlock + g;
  __shared__ float red[8];
  const bool active = row < M;
  const int nchunk = K >> 3;  // 8 elements per 16-byte chunk

  uint4 raw[CHUNKS];
  AbsMax2<T> running;
  if (active) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * ldx);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int idx = c * G + t;
      raw[c] = idx < nchunk ? __ldg(src + idx) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      running.add(raw[c].x);
      running.add(raw[c].y);
      running.add(raw[c].z);
      running.add(raw[c].w);
    }
  }
  float amax = warp_max(running.value());
  if (G > 32) {
    // the row's G/32 warps are neighbours in the block: combine their maxima
    constexpr int kWarpsPerRow = G / 32;
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    float m = red[g * kWarpsPerRow];
#pragma unroll
    for (int i = 1; i < kWarpsPerRow; ++i) m = fmaxf(m, red[g * kWarpsPerRow + i]);
    amax = m;
  }
  if (!active) return;
  const float scale = fmaxf(__fdiv_rn(amax, 127.0f), 1e-8f);
  const float inv_scale = __frcp_rn(scale);
  if (t == 0) a_scales[row] = scale;
  uint2* dst = reinterpret_cast<uint2*>(xq + static_cast<size_t>(row) * K);
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int idx = c * G + t;
    if (idx < nchunk) dst[idx] = quant8<T>(raw[c], scale, inv_scale);
  }
}

// Any K: one 256-thread CTA per row, the row is read twice (the second read hits L2).
template <typename T>
__global__ void __launch_bounds__(256)
act_quant_long_rows_kernel(const T* __restrict__ x, int64_t ldx, int8_t* __restrict__ xq,
                           float* __restrict__ a_scales, int M, int K) {
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  const int row = blockIdx.x;
  __shared__ float red[8];
  const int nchunk = K >> 3;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * ldx);
  AbsMax2<T> running;
  for (int idx = threadIdx.x; idx < nchunk; idx += 256) {
    const uint4 r = __ldg(src + idx);
    running.add(r.x);
    running.add(r.y);
    running.add(r.z);
    running.add(r.w);
  }
  float amax = warp_max(running.value());
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  float m = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
  const float scale = fmaxf(__fdiv_rn(m, 127.0f), 1e-8f);
  const float inv_scale = __frcp_rn(scale);
  if (threadIdx.x == 0) a_scales[row] = scale;
  uint2* dst = reinterpret_cast<uint2*>(xq + static_cast<size_t>(row) * K);
  for (int idx = threadIdx.x; idx < nchunk; idx += 256)
    dst[idx] = quant8<T>(__ldg(src + idx), scale, inv_scale);
}

template <typename T>
cudaError_t launch_typed(const T* x, int64_t ldx, int8_t* xq, float* a_scales, int M, int K,
                         cudaStream_t s) {
  // Four 16-byte chunks per thread keep the register count low (high occupancy); longer
  // rows are spread over more threads instead of more chunks.
  auto blocks = [&](int g) { return (M + (256 / g) - 1) / (256 / g); };
  if (K <= 32 * 8 * 2) {
    return launch_overlapped(act_quant_rows_kernel<T, 32, 2>, blocks(32), 256, 0, s, x, ldx, xq, a_scales, M, K);
  } else if (K <= 32 * 8 * 4) {
    return launch_overlapped(act_quant_rows_kernel<T, 32, 4>, blocks(32), 256, 0, s, x, ldx, xq, a_scales, M, K);
  } else if (K <= 64 * 8 * 4) {
    return launch_overlapped(act_quant_rows_kernel<T, 64, 4>, blocks(64), 256, 0, s, x, ldx, xq, a_scales, M, K);
  } else if (K <= 128 * 8 * 4) {
    return launch_overlapped(act_quant_rows_kernel<T, 128, 4>, blocks(128), 256, 0, s, x, ldx, xq, a_scales, M, K);
  } else if (K <= 256 * 8 * 4) {
    return launch_overlapped(act_quant_rows_kernel<T, 256, 4>, blocks(256), 256, 0, s, x, ldx, xq, a_scales, M, K);
  } else if (K <= 256 * 8 * 8) {
    return launch_overlapped(act_quant_rows_kernel<T, 256, 8>, blocks(256), 256, 0, s, x, ldx, xq, a_scales, M, K);
  } else {
    return launch_overlapped(act_quant_long_rows_kernel<T>, M, 256, 0, s, x, ldx, xq, a_scales, M, K);
  }
}

}  // namespace

cudaError_t launch_act_quant(const void* x, int64_t ldx, int x_dtype, int8_t* xq, float* a_scales,
                             int M, int K, cudaStream_t stream) {
  cudaError_t e;
  if (x_dtype == B200Q_DTYPE_BF16) {
    e = launch_typed(reinterpret_cast<const __nv_bfloat16*>(x), ldx, xq, a_scales, M, K, stream);
  } else {
    e = launch_typed(reinterpret_cast<const __half*>(x), ldx, xq, a_scales, M, K, stream);
  }
  if (e == cudaSuccess) count_launch();
  return e;
}

}  // namespace b200q
