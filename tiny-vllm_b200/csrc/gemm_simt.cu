// Weight-streaming SIMT kernels for very small token counts (and as an independent
// second implementation the tensor-core kernels are cross-checked against).
//
// One warp owns one output channel n: its 32 lanes walk the weight row qweight[n,:]
// with 128-bit loads, each lane dots its 16 int8 weights against the matching slice
// of up to MT token rows, and the lanes' partial sums are combined with warp
// shuffles.  Weights are read once per group of MT tokens, activations come from L1/L2.
//
//   W8A8 : int32 dp4a accumulation, then (float(acc) * a_s[m]) * w_s[n] + bias[n]
//          (nanovllm/quantization/csrc/w8a8_gemm.cu:165-183 and :195-200)
//   W8A16: fp32 accumulation of x[m,k] * float(q[n,k]), then acc * s[n] + bias[n]
//          (nanovllm/quantization/csrc/int8_weight_only_gemm.cu:258-292 computes the
//          same sum with the scale applied per product)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.h"

namespace b200q {
namespace {

constexpr int kWarps = 8;  // channels per block
constexpr int kMT = 8;     // token rows per pass

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ __half from_float<__half>(float v) {
  return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<__half>(__half v) {
  return __half2float(v);
}
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t u);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) {
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t u) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

template <typename OutT, bool RAW_I32>
__global__ void __launch_bounds__(kWarps * 32)
w8a8_stream_kernel(const int8_t* __restrict__ xq, const int8_t* __restrict__ w,
                   const float* __restrict__ a_s, const float* __restrict__ w_s,
                   const OutT* __restrict__ bias, void* __restrict__ out, int M, int N, int K) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kWarps + warp;
  if (n >= N) return;
  const int m0 = blockIdx.y * kMT;
  const int rows = min(kMT, M - m0);
  int acc[kMT];
#pragma unroll
  for (int i = 0; i < kMT; ++i) acc[i] = 0;
  const int4* wrow = reinterpret_cast<const int4*>(w + static_cast<size_t>(n) * K);
  const int nchunk = K >> 4;
  for (int c = lane; c < nchunk; c += 32) {
    const int4 wv = __ldg(wrow + c);
#pragma unroll
    for (int i = 0; i < kMT; ++i) {
      if (i < rows) {
        const int4 xv =
            __ldg(reinterpret_cast<const int4*>(xq + static_cast<size_t>(m0 + i) * K) + c);
        int a = acc[i];
        a = __dp4a(wv.x, xv.x, a);
        a = __dp4a(wv.y, xv.y, a);
        a = __dp4a(wv.z, xv.z, a);
        a = __dp4a(wv.w, xv.w, a);
        acc[i] = a;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kMT; ++i) acc[i] = warp_sum(acc[i]);
  if (lane == 0) {
    for (int i = 0; i < rows; ++i) {
      const size_t o = static_cast<size_t>(m0 + i) * N + n;
      if (RAW_I32) {
        reinterpret_cast<int32_t*>(out)[o] = acc[i];
      } else {
        const float b = bias != nullptr ? to_float<OutT>(bias[n]) : 0.f;
        const float v =
            __fadd_rn(__fmul_rn(__fmul_rn(static_cast<float>(acc[i]), a_s[m0 + i]), w_s[n]), b);
        reinterpret_cast<OutT*>(out)[o] = from_float<OutT>(v);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
w8a16_stream_kernel(const T* __restrict__ x, const int8_t* __restrict__ w,
                    const float* __restrict__ s, const T* __restrict__ bias, T* __restrict__ y,
                    int M, int N, int K) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kWarps + warp;
  if (n >= N) return;
  const int m0 = blockIdx.y * kMT;
  const int rows = min(kMT, M - m0);
  float acc[kMT];
#pragma unroll
  for (int i = 0; i < kMT; ++i) acc[i] = 0.f;
  const int4* wrow = reinterpret_cast<const int4*>(w + static_cast<size_t>(n) * K);
  const int nchunk = K >> 4;
  for (int c = lane; c < nchunk; c += 32) {
    const int4 wv = __ldg(wrow + c);
    float wf[16];
    const int wi[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      wf[4 * j + 0] = static_cast<float>(static_cast<int8_t>(wi[j] & 0xFF));
      wf[4 * j + 1] = static_cast<float>(static_cast<int8_t>((wi[j] >> 8) & 0xFF));
      wf[4 * j + 2] = static_cast<float>(static_cast<int8_t>((wi[j] >> 16) & 0xFF));
      wf[4 * j + 3] = static_cast<float>(static_cast<int8_t>((wi[j] >> 24) & 0xFF));
    }
#pragma unroll
    for (int i = 0; i < kMT; ++i) {
      if (i < rows) {
        const uint4* xp =
            reinterpret_cast<const uint4*>(x + static_cast<size_t>(m0 + i) * K) + 2 * c;
        const uint4 x0 = __ldg(xp), x1 = __ldg(xp + 1);
        const uint32_t xu[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        float a = acc[i];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 xf = unpack2<T>(xu[j]);
          a = fmaf(xf.x, wf[2 * j], a);
          a = fmaf(xf.y, wf[2 * j + 1], a);
        }
        acc[i] = a;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kMT; ++i) acc[i] = warp_sum(acc[i]);
  if (lane == 0) {
    const float sc = s[n];
    const float b = bias != nullptr ? to_float<T>(bias[n]) : 0.f;
    for (int i = 0; i < rows; ++i)
      y[static_cast<size_t>(m0 + i) * N + n] = from_float<T>(__fadd_rn(__fmul_rn(acc[i], sc), b));
  }
}

}  // namespace

cudaError_t launch_w8a8_simt(const GemmArgs& a) {
  dim3 grid((a.N + kWarps - 1) / kWarps, (a.M + kMT - 1) / kMT);
  if (grid.y > 65535) return cudaErrorInvalidConfiguration;
  const int8_t* xq = reinterpret_cast<const int8_t*>(a.x);
  if (a.acc_out != nullptr) {
    w8a8_stream_kernel<__nv_bfloat16, true><<<grid, kWarps * 32, 0, a.stream>>>(
        xq, a.w, nullptr, nullptr, nullptr, a.acc_out, a.M, a.N, a.K);
  } else if (a.dtype == B200Q_DTYPE_BF16) {
    w8a8_stream_kernel<__nv_bfloat16, false><<<grid, kWarps * 32, 0, a.stream>>>(
        xq, a.w, a.a_scales, a.w_scales, reinterpret_cast<const __nv_bfloat16*>(a.bias), a.y, a.M,
        a.N, a.K);
  } else {
    w8a8_stream_kernel<__half, false><<<grid, kWarps * 32, 0, a.stream>>>(
        xq, a.w, a.a_scales, a.w_scales, reinterpret_cast<const __half*>(a.bias), a.y, a.M, a.N,
        a.K);
  }
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) count_launch();
  return e;
}

cudaError_t launch_w8a16_simt(const GemmArgs& a) {
  dim3 grid((a.N + kWarps - 1) / kWarps, (a.M + kMT - 1) / kMT);
  if (grid.y > 65535) return cudaErrorInvalidConfiguration;
  if (a.dtype == B200Q_DTYPE_BF16) {
    w8a16_stream_kernel<__nv_bfloat16><<<grid, kWarps * 32, 0, a.stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(a.x), a.w, a.w_scales,
        reinterpret_cast<const __nv_bfloat16*>(a.bias), reinterpret_cast<__nv_bfloat16*>(a.y), a.M,
        a.N, a.K);
  } else {
    w8a16_stream_kernel<__half><<<grid, kWarps * 32, 0, a.stream>>>(
        reinterpret_cast<const __half*>(a.x), a.w, a.w_scales,
        reinterpret_cast<const __half*>(a.bias), reinterpret_cast<__half*>(a.y), a.M, a.N, a.K);
  }
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) count_launch();
  return e;
}

}  // namespace b200q
