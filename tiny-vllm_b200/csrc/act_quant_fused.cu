// Per-token int8 quantisation fused into the two operations that produce the inputs of the
// W8A8 linear layers, so that the 16-bit activation never makes a round trip through HBM:
//
//   add-RMSNorm -> quant   feeds qkv_proj and gate_up_proj
//       (nanovllm/layers/layernorm.py:16-40, called from nanovllm/models/qwen3.py:160-166)
//       s      = float(x) + float(residual)                     (residual optional)
//       res'   = T(s)
//       var    = mean_k s^2
//       n      = T(s * rsqrt(var + eps))
//       y      = T(n * weight)                                   (16-bit multiply, one rounding)
//   SiLU-mul -> quant      feeds down_proj
//       (nanovllm/layers/activation.py:11-14, called from nanovllm/models/qwen3.py:119-121)
//       y      = T(silu(float(gate)) * float(up)),  [gate | up] = the two halves of a row
//
// followed, on the 16-bit values y held in registers, by exactly the arithmetic of the
// stand-alone quantiser (nanovllm/quantization/utils.py:28-32): the int8 codes and scales
// are bit-identical to quantising the y this kernel would have written.  y itself is
// written only on request.
//
// A row is owned by G threads (32..256), each holding CHUNKS 16-byte chunks in registers,
// like act_quant_rows_kernel; rows longer than 16384 elements are not taken.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <climits>

#include "act_quant_device.cuh"
#include "common.h"
#include "ptx_sm100.cuh"

namespace b200q {
namespace {

template <typename T, int G, int CHUNKS>
__global__ void __launch_bounds__(256)
add_rmsnorm_quant_kernel(const T* __restrict__ x, const T* residual_in, const T* __restrict__ weight,
                         float eps, T* residual_out, T* __restrict__ y_out, int8_t* __restrict__ xq,
                         float* __restrict__ a_scales, int M, int K) {
  constexpr int kRowsPerBlock = 256 / G;
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  const int g = threadIdx.x / G, t = threadIdx.x % G;
  const int row = blockIdx.x * kRowsPerBlock + g;
  __shared__ float red[8];
  const bool active = row < M;
  const int nchunk = K >> 3;

  float s[CHUNKS][8];
  float sumsq = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int idx = c * G + t;
    const bool live = active && idx < nchunk;
    uint4 xv = make_uint4(0u, 0u, 0u, 0u), rv = xv;
    if (live) {
      xv = __ldg(reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * K) + idx);
      if (residual_in != nullptr)
        rv = *(reinterpret_cast<const uint4*>(residual_in + static_cast<size_t>(row) * K) + idx);
    }
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, rw[4] = {rv.x, rv.y, rv.z, rv.w};
    uint32_t out[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = unpack2<T>(xw[i]), b = unpack2<T>(rw[i]);
      const float s0 = residual_in != nullptr ? __fadd_rn(a.x, b.x) : a.x;
      const float s1 = residual_in != nullptr ? __fadd_rn(a.y, b.y) : a.y;
      s[c][2 * i] = s0;
      s[c][2 * i + 1] = s1;
      sumsq = __fmaf_rn(s0, s0, sumsq);
      sumsq = __fmaf_rn(s1, s1, sumsq);
      out[i] = pack2<T>(s0, s1);
    }
    if (live && residual_out != nullptr)
      *(reinterpret_cast<uint4*>(residual_out + static_cast<size_t>(row) * K) + idx) =
          make_uint4(out[0], out[1], out[2], out[3]);
  }
  const float total = group_reduce<G, false>(sumsq, red, g);
  const float inv_rms = __frsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(K)), eps));

  uint4 y[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int idx = c * G + t;
    uint4 wv = make_uint4(0u, 0u, 0u, 0u);
    if (idx < nchunk) wv = __ldg(reinterpret_cast<const uint4*>(weight) + idx);
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
    uint32_t out[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t n = pack2<T>(__fmul_rn(s[c][2 * i], inv_rms), __fmul_rn(s[c][2 * i + 1], inv_rms));
      out[i] = mul2_16<T>(n, ww[i]);
    }
    y[c] = make_uint4(out[0], out[1], out[2], out[3]);
  }
  quantise_row<T, G, CHUNKS>(y, active, row, t, g, nchunk, K, y_out, xq, a_scales, red);
}

// silu(v) = v / (1 + e^-v) with the hardware exponential and reciprocal (relative error about
// 2e-7): the result is rounded to 8 or 11 significant bits next, so one element in several
// thousand lands on the neighbouring 16-bit value compared with a correctly rounded silu; an
// IEEE division and expf made the kernel instruction-bound (52 us instead of the 25 us its
// 126 MB take at M = 8192, I = 3072).
__device__ __forceinline__ float silu(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

// gate_up: [M, ld] with the gate in columns [0, I) and the up projection in [I, 2 I).
template <typename T, int G, int CHUNKS>
__global__ void __launch_bounds__(256)
silu_mul_quant_kernel(const T* __restrict__ gate_up, int64_t ld, T* __restrict__ y_out,
                      int8_t* __restrict__ xq, float* __restrict__ a_scales, int M, int I) {
  constexpr int kRowsPerBlock = 256 / G;
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  const int g = threadIdx.x / G, t = threadIdx.x % G;
  const int row = blockIdx.x * kRowsPerBlock + g;
  __shared__ float red[8];
  const bool active = row < M;
  const int nchunk = I >> 3;

  uint4 y[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int idx = c * G + t;
    uint4 gv = make_uint4(0u, 0u, 0u, 0u), uv = gv;
    if (active && idx < nchunk) {
      const uint4* base = reinterpret_cast<const uint4*>(gate_up + static_cast<size_t>(row) * ld);
      gv = __ldg(base + idx);
      uv = __ldg(base + nchunk + idx);
    }
    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
    uint32_t out[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = unpack2<T>(gw[i]), b = unpack2<T>(uw[i]);
      out[i] = pack2<T>(__fmul_rn(silu(a.x), b.x), __fmul_rn(silu(a.y), b.y));
    }
    y[c] = make_uint4(out[0], out[1], out[2], out[3]);
  }
  quantise_row<T, G, CHUNKS>(y, active, row, t, g, nchunk, I, y_out, xq, a_scales, red);
}

// Picks the row-group width for a row of K elements and launches; false = row too long.
#define B200Q_FUSED_DISPATCH(KERNEL, KLEN, ...)                                              \
  do {                                                                                       \
    auto blocks = [&](int g) { return (M + (256 / g) - 1) / (256 / g); };                     \
    if ((KLEN) <= 32 * 8 * 4)                                                                \
      e = launch_overlapped(KERNEL<T, 32, 4>, blocks(32), 256, 0, st, __VA_ARGS__);          \
    else if ((KLEN) <= 64 * 8 * 4)                                                           \
      e = launch_overlapped(KERNEL<T, 64, 4>, blocks(64), 256, 0, st, __VA_ARGS__);          \
    else if ((KLEN) <= 128 * 8 * 4)                                                          \
      e = launch_overlapped(KERNEL<T, 128, 4>, blocks(128), 256, 0, st, __VA_ARGS__);        \
    else if ((KLEN) <= 256 * 8 * 4)                                                          \
      e = launch_overlapped(KERNEL<T, 256, 4>, blocks(256), 256, 0, st, __VA_ARGS__);        \
    else                                                                                     \
      e = launch_overlapped(KERNEL<T, 256, 8>, blocks(256), 256, 0, st, __VA_ARGS__);        \
  } while (0)

template <typename T>
cudaError_t launch_rmsnorm(const void* x, const void* res_in, const void* weight, float eps,
                           void* res_out, void* y, int8_t* xq, float* a_s, int M, int K,
                           cudaStream_t st) {
  cudaError_t e;
  B200Q_FUSED_DISPATCH(add_rmsnorm_quant_kernel, K, static_cast<const T*>(x),
                       static_cast<const T*>(res_in), static_cast<const T*>(weight), eps,
                       static_cast<T*>(res_out), static_cast<T*>(y), xq, a_s, M, K);
  return e;
}

template <typename T>
cudaError_t launch_silu(const void* gate_up, int64_t ld, void* y, int8_t* xq, float* a_s, int M,
                        int I, cudaStream_t st) {
  cudaError_t e;
  B200Q_FUSED_DISPATCH(silu_mul_quant_kernel, I, static_cast<const T*>(gate_up), ld,
                       static_cast<T*>(y), xq, a_s, M, I);
  return e;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace b200q

extern "C" int b200q_add_rmsnorm_quant_i8(const void* x, const void* residual_in, const void* weight,
                                          float eps, void* residual_out, void* y, int8_t* xq,
                                          float* a_scales, int M, int K, int dtype, void* stream) {
  using namespace b200q;
  if (x == nullptr || weight == nullptr || xq == nullptr || a_scales == nullptr)
    return B200Q_ERR_NULL_POINTER;
  if (M <= 0 || K <= 0 || static_cast<long long>(M) * K > INT_MAX) return B200Q_ERR_BAD_SHAPE;
  if (dtype != B200Q_DTYPE_F16 && dtype != B200Q_DTYPE_BF16) return B200Q_ERR_BAD_ARGUMENT;
  if ((K % 16) != 0 || K > 256 * 8 * 8) return B200Q_ERR_UNSUPPORTED_SHAPE;
  if (!aligned16(x) || !aligned16(weight) || !aligned16(xq) || !aligned16(residual_in) ||
      !aligned16(residual_out) || !aligned16(y) || (reinterpret_cast<uintptr_t>(a_scales) & 3u) != 0)
    return B200Q_ERR_MISALIGNED;
  if (device_cc_major() != 10) return B200Q_ERR_UNSUPPORTED_ARCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = dtype == B200Q_DTYPE_BF16
                      ? launch_rmsnorm<__nv_bfloat16>(x, residual_in, weight, eps, residual_out, y, xq,
                                                      a_scales, M, K, st)
                      : launch_rmsnorm<__half>(x, residual_in, weight, eps, residual_out, y, xq,
                                               a_scales, M, K, st);
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch();
  return B200Q_OK;
}

extern "C" int b200q_silu_mul_quant_i8(const void* gate_up, int64_t ld, void* y, int8_t* xq,
                                       float* a_scales, int M, int I, int dtype, void* stream) {
  using namespace b200q;
  if (gate_up == nullptr || xq == nullptr || a_scales == nullptr) return B200Q_ERR_NULL_POINTER;
  if (M <= 0 || I <= 0 || static_cast<long long>(M) * I * 2 > INT_MAX) return B200Q_ERR_BAD_SHAPE;
  if (dtype != B200Q_DTYPE_F16 && dtype != B200Q_DTYPE_BF16) return B200Q_ERR_BAD_ARGUMENT;
  if ((I % 16) != 0 || I > 256 * 8 * 8 || ld < 2 * static_cast<int64_t>(I) || (ld % 8) != 0)
    return B200Q_ERR_UNSUPPORTED_SHAPE;
  if (!aligned16(gate_up) || !aligned16(xq) || !aligned16(y) ||
      (reinterpret_cast<uintptr_t>(a_scales) & 3u) != 0)
    return B200Q_ERR_MISALIGNED;
  if (device_cc_major() != 10) return B200Q_ERR_UNSUPPORTED_ARCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = dtype == B200Q_DTYPE_BF16
                      ? launch_silu<__nv_bfloat16>(gate_up, ld, y, xq, a_scales, M, I, st)
                      : launch_silu<__half>(gate_up, ld, y, xq, a_scales, M, I, st);
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch();
  return B200Q_OK;
}
