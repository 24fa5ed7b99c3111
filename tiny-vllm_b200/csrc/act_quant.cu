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

#include "act_quant_device.cuh"
#include "common.h"
#include "ptx_sm100.cuh"

namespace b200q {
namespace {

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
