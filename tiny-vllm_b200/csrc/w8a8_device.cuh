// Device-side pieces shared by the W8A8 tcgen05 kernels (single-CTA and CTA-pair):
// tile constants, kernel parameters, and the epilogue arithmetic
// (float(acc) * a_scale) * w_scale + bias of nanovllm/quantization/csrc/w8a8_gemm.cu:387-390.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200q {
namespace {

constexpr int kTileA = 128;       // UMMA M
constexpr int kBlockK = 128;      // bytes of K per pipeline stage = one swizzle row
constexpr int kUmmaK = 32;        // bytes of K per tcgen05.mma kind::i8
constexpr int kEpiWarps = 8;      // warps 2..9: two per TMEM lane quarter
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kThreads = 64 + kEpiThreads;  // + warp 0 (TMA) + warp 1 (UMMA)
constexpr int kSlabBytes = 32 * 128;         // per-warp transpose buffer: 32 rows x 64 cols x 2 B
constexpr int kStagingBytes = kEpiWarps * kSlabBytes;
constexpr int kScaleSmemBytes = 2 * 256 * 4;  // channel scales of the current tile, double-buffered
constexpr int kCtrlBytes = 256;
constexpr int kMaxStages = 8;
constexpr int kMaxSmem = 227 * 1024;

enum { OUT_SCALED = 0, OUT_I32 = 1 };

struct KernelParams {
  int rows_a, rows_b;
  int bn;
  int tiles_a, tiles_b;
  int k_blocks, splits, kb_per_split;
  int stages;
  int cluster;             // CTAs per cluster splitting K (1 = off); split index = cluster rank
  int partial_bytes;       // shared memory the cluster leader receives partial tiles in
  int tmem_cols;
  int swap;
  int n_channels;          // leading dimension of the output
  int n_tokens;
  const float* a_scales;   // per token
  const float* w_scales;   // per channel
  const void* bias;        // per channel, OutT
  void* out;               // OutT [M,N] or int32 [M,N]
  int32_t* partials;
  unsigned int* counters;
  int* status;
  int debug_flags;         // test-only: 1 = skip epilogue work, 2 = skip UMMA issue
  int fast_store;          // 1: 16-bit outputs are transposed through shared memory and stored as full 128-byte rows
};

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
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  T a = from_float<T>(lo), b = from_float<T>(hi);
  uint16_t ua = *reinterpret_cast<uint16_t*>(&a), ub = *reinterpret_cast<uint16_t*>(&b);
  return static_cast<uint32_t>(ua) | (static_cast<uint32_t>(ub) << 16);
}

// (acc * a_scale) * w_scale + bias with one rounding per operation, as the
// reference epilogue is written (no fused multiply-add).
__device__ __forceinline__ float scale_acc(int acc, float a_s, float w_s, float b) {
  return __fadd_rn(__fmul_rn(__fmul_rn(static_cast<float>(acc), a_s), w_s), b);
}

// Writes the 32 accumulators this thread holds for columns [c0, c0+32) of its row.
template <typename OutT, int MODE>
__device__ __forceinline__ void emit_chunk(const KernelParams& p, int tile_a, int tile_b,
                                           int row_in_tile, int c0, const uint32_t (&v)[32]) {
  const int row_a = tile_a * kTileA + row_in_tile;
  const int col_b0 = tile_b * p.bn + c0;
  if (row_a >= p.rows_a || col_b0 >= p.rows_b) return;
  const int N = p.n_channels;
  if (!p.swap) {
    // row = token, columns = channels: the thread owns 32 consecutive outputs of a row.
    const size_t off = static_cast<size_t>(row_a) * N + col_b0;
    const bool full = (col_b0 + 32 <= p.rows_b);
    if (MODE == OUT_I32) {
      int32_t* dst = reinterpret_cast<int32_t*>(p.out) + off;
      if (full && (N & 3) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<uint4*>(dst + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col_b0 + j < p.rows_b) dst[j] = static_cast<int32_t>(v[j]);
      }
    } else {
      const float a_s = __ldg(p.a_scales + row_a);
      const OutT* bias = reinterpret_cast<const OutT*>(p.bias);
      OutT* dst = reinterpret_cast<OutT*>(p.out) + off;
      if (full && (N & 7) == 0) {
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 ws = __ldg(reinterpret_cast<const float4*>(p.w_scales + col_b0 + j));
          float b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
          if (bias != nullptr) {
            b0 = to_float<OutT>(bias[col_b0 + j]);
            b1 = to_float<OutT>(bias[col_b0 + j + 1]);
            b2 = to_float<OutT>(bias[col_b0 + j + 2]);
            b3 = to_float<OutT>(bias[col_b0 + j + 3]);
          }
          packed[j / 2] = pack2<OutT>(scale_acc(static_cast<int>(v[j]), a_s, ws.x, b0),
                                      scale_acc(static_cast<int>(v[j + 1]), a_s, ws.y, b1));
          packed[j / 2 + 1] = pack2<OutT>(scale_acc(static_cast<int>(v[j + 2]), a_s, ws.z, b2),
                                          scale_acc(static_cast<int>(v[j + 3]), a_s, ws.w, b3));
        }
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          *reinterpret_cast<uint4*>(reinterpret_cast<uint32_t*>(dst) + j) =
              make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (col_b0 + j < p.rows_b) {
            const float b = bias != nullptr ? to_float<OutT>(bias[col_b0 + j]) : 0.f;
            dst[j] = from_float<OutT>(
                scale_acc(static_cast<int>(v[j]), a_s, __ldg(p.w_scales + col_b0 + j), b));
          }
        }
      }
    }
  } else {
    // row = channel, columns = tokens: consecutive lanes write consecutive channels.
    if (MODE == OUT_I32) {
      int32_t* dst = reinterpret_cast<int32_t*>(p.out);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int tok = col_b0 + j;
        if (tok < p.rows_b) dst[static_cast<size_t>(tok) * N + row_a] = static_cast<int32_t>(v[j]);
      }
    } else {
      const float w_s = __ldg(p.w_scales + row_a);
      const OutT* bias = reinterpret_cast<const OutT*>(p.bias);
      const float b = bias != nullptr ? to_float<OutT>(bias[row_a]) : 0.f;
      OutT* dst = reinterpret_cast<OutT*>(p.out);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int tok = col_b0 + j;
        if (tok < p.rows_b) {
          const float a_s = __ldg(p.a_scales + tok);
          dst[static_cast<size_t>(tok) * N + row_a] =
              from_float<OutT>(scale_acc(static_cast<int>(v[j]), a_s, w_s, b));
        }
      }
    }
  }
}

template <typename T>
__device__ __forceinline__ uint32_t pack2_rn(float2 v);
template <>
__device__ __forceinline__ uint32_t pack2_rn<__nv_bfloat16>(float2 v) {
  const __nv_bfloat162 h = __float22bfloat162_rn(v);  // one cvt.rn.bf16x2.f32
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2_rn<__half>(float2 v) {
  const __half2 h = __float22half2_rn(v);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// 32 accumulators of one row -> 16 packed 16-bit pairs, written to this thread's row of
// the warp's transpose buffer (rows of 128 bytes, 16-byte chunk c of row r stored at
// chunk c ^ (r & 7) so that both the row-wise writes and the later reads are free of
// bank conflicts).  Packed fp32x2 arithmetic (mul.f32x2 / add.f32x2 round each half like
// the scalar instruction, so results are unchanged): (acc * a_s) * w_s [+ bias].
template <typename OutT, bool HAS_BIAS>
__device__ __forceinline__ void convert_chunk(const KernelParams& p, const float* s_ws, float a_s,
                                              int col0, int lane, int chunk_half, uint8_t* slab,
                                              const uint32_t (&v)[32]) {
  const OutT* bias = reinterpret_cast<const OutT*>(p.bias);
  const float2 a2 = make_float2(a_s, a_s);
  uint32_t packed[16];
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 ws = *reinterpret_cast<const float4*>(s_ws + j);
    float2 lo = make_float2(static_cast<float>(static_cast<int>(v[j])),
                            static_cast<float>(static_cast<int>(v[j + 1])));
    float2 hi = make_float2(static_cast<float>(static_cast<int>(v[j + 2])),
                            static_cast<float>(static_cast<int>(v[j + 3])));
    lo = __fmul2_rn(__fmul2_rn(lo, a2), make_float2(ws.x, ws.y));
    hi = __fmul2_rn(__fmul2_rn(hi, a2), make_float2(ws.z, ws.w));
    if (HAS_BIAS) {
      float b[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        b[u] = col0 + j + u < p.rows_b ? to_float<OutT>(bias[col0 + j + u]) : 0.f;
      // scalar adds: __fadd_rn is never contracted with the multiply before it (the
      // packed add was seen fused into an fma.f32x2, one rounding instead of two)
      lo = make_float2(__fadd_rn(lo.x, b[0]), __fadd_rn(lo.y, b[1]));
      hi = make_float2(__fadd_rn(hi.x, b[2]), __fadd_rn(hi.y, b[3]));
    }
    packed[j / 2] = pack2_rn<OutT>(lo);
    packed[j / 2 + 1] = pack2_rn<OutT>(hi);
  }
  const int sw = lane & 7;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int chunk = chunk_half * 4 + c;  // 16-byte chunk index inside the 128-byte row
    *reinterpret_cast<uint4*>(slab + lane * 128 + ((chunk ^ sw) << 4)) =
        make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
  }
}

// Reads the warp's 32 x 64 transpose buffer back row-wise (8 lanes per 128-byte row) and
// stores full rows: every store instruction writes four complete 128-byte lines.
template <typename OutT>
__device__ __forceinline__ void store_group(const KernelParams& p, const uint8_t* slab, int lane,
                                            int row0, int col0) {
  const int c = lane & 7;
  const int col = col0 + c * 8;
  OutT* out = reinterpret_cast<OutT*>(p.out);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3);
    const uint4 val = *reinterpret_cast<const uint4*>(slab + r * 128 + ((c ^ (r & 7)) << 4));
    const int row = row0 + r;
    if (row < p.rows_a && col < p.rows_b)  // N % 8 == 0: a 16-byte piece is all in or all out
      *reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * p.n_channels + col) = val;
  }
}

}  // namespace
}  // namespace b200q
