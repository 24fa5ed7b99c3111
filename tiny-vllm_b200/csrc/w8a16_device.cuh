// Device-side pieces shared by the W8A16 tcgen05 kernels (single-CTA and CTA-pair): tile
// constants, kernel parameters, exact int8 -> 16-bit expansion into the swizzled operand
// layout, and the epilogue arithmetic acc * s[n] + b[n].
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200q {
namespace {

constexpr int kTileA = 128;        // UMMA M
constexpr int kBlockK = 64;        // K elements per pipeline stage
constexpr int kRow16 = 128;        // bytes of one row of a 16-bit operand tile (= swizzle row)
constexpr int kRow8 = 64;          // bytes of one row of the raw int8 tile
constexpr int kUmmaK = 16;         // K elements per tcgen05.mma kind::f16
constexpr int kEpiWarps = 4;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kConvWarps = 8;      // two per scheduler: the expansion is latency-bound per warp
constexpr int kConvThreads = kConvWarps * 32;
constexpr int kThreads = 64 + kEpiThreads + kConvThreads;
constexpr int kMaxConvBufs = 8;    // ring of converted tiles: 2 for 256-row tiles, more for narrow ones
constexpr int kMaxStages = 8;
constexpr int kMaxSmem = 227 * 1024;
constexpr int kSlabBytes = 32 * 128;  // per-epilogue-warp transpose buffer (32 rows x 64 cols x 2 B)
constexpr int kStagingBytes = kEpiWarps * kSlabBytes;
constexpr int kScaleSmemBytes = 2 * 256 * 4;
constexpr int kCtrlBytes = 512;

struct KernelParams {
  int rows_a, rows_b;
  int bn;
  int tiles_a, tiles_b;
  int k_blocks, splits, kb_per_split;
  int stages;
  int conv_bufs;
  int cluster;        // CTAs per cluster splitting K (1 = off); split index = cluster rank
  int partial_bytes;  // shared memory the cluster leader receives partial tiles in
  int tmem_cols;
  int swap;
  int n_channels;
  int is_bf16;
  const float* w_scales;
  const void* bias;
  void* out;
  float* partials;
  unsigned int* counters;
  int* status;
  int fast_store;
  int debug_flags;
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
__device__ __forceinline__ uint32_t pack2_rn(float2 v);
template <>
__device__ __forceinline__ uint32_t pack2_rn<__nv_bfloat16>(float2 v) {
  const __nv_bfloat162 h = __float22bfloat162_rn(v);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2_rn<__half>(float2 v) {
  const __half2 h = __float22half2_rn(v);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// ------------------------------------------------------------ int8 -> 16-bit expansion
// Four int8 (one 32-bit word) -> four values of type T, exact.
//   fp16: 0x6400 | u is the half 1024 + u (u = q + 128 in 0..255); subtract 1152.
//   bf16: 0x4B000000 | u is the float 2^23 + u; subtract 2^23 + 128; the result has at
//         most 8 significant bits, so the conversion to bf16 is exact.
template <typename T>
__device__ __forceinline__ uint2 expand4(uint32_t w);
template <>
__device__ __forceinline__ uint2 expand4<__half>(uint32_t w) {
  const uint32_t t = w ^ 0x80808080u;
  uint32_t lo = __byte_perm(t, 0x64646464u, 0x4140);
  uint32_t hi = __byte_perm(t, 0x64646464u, 0x4342);
  const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
  const __half2 l = __hsub2(*reinterpret_cast<__half2*>(&lo), bias);
  const __half2 h = __hsub2(*reinterpret_cast<__half2*>(&hi), bias);
  return make_uint2(*reinterpret_cast<const uint32_t*>(&l), *reinterpret_cast<const uint32_t*>(&h));
}
template <>
__device__ __forceinline__ uint2 expand4<__nv_bfloat16>(uint32_t w) {
  const uint32_t t = w ^ 0x80808080u;
  const float2 magic = make_float2(-8388736.f, -8388736.f);  // -(2^23 + 128)
  const float2 f01 = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(t, 0x4B000000u, 0x7540)),
                                            __uint_as_float(__byte_perm(t, 0x4B000000u, 0x7541))),
                                magic);
  const float2 f23 = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(t, 0x4B000000u, 0x7542)),
                                            __uint_as_float(__byte_perm(t, 0x4B000000u, 0x7543))),
                                magic);
  // the sums are integers of at most 8 significant bits: their bf16 form is the upper half of
  // the fp32 word, taken with a byte permute (the packing conversion runs on a slower pipe)
  return make_uint2(__byte_perm(__float_as_uint(f01.x), __float_as_uint(f01.y), 0x7632),
                    __byte_perm(__float_as_uint(f23.x), __float_as_uint(f23.y), 0x7632));
}

// One row (64 int8) of the raw tile -> one row (128 bytes) of the 16-bit tile.
//   raw tile : rows of 64 bytes, 64-byte swizzle  (chunk c of row r at c ^ ((r >> 1) & 3))
//   16-bit   : rows of 128 bytes, 128-byte swizzle (chunk c of row r at c ^ (r & 7))
template <typename T>
__device__ __forceinline__ void expand_row(const uint8_t* raw, uint8_t* dst, int r) {
  const uint8_t* src_row = raw + r * kRow8;
  uint8_t* dst_row = dst + r * kRow16;
  const int sw8 = (r >> 1) & 3;
  const int sw16 = r & 7;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint4 w = *reinterpret_cast<const uint4*>(src_row + ((c ^ sw8) << 4));
    const uint2 e0 = expand4<T>(w.x), e1 = expand4<T>(w.y), e2 = expand4<T>(w.z),
                e3 = expand4<T>(w.w);
    *reinterpret_cast<uint4*>(dst_row + (((2 * c) ^ sw16) << 4)) = make_uint4(e0.x, e0.y, e1.x, e1.y);
    *reinterpret_cast<uint4*>(dst_row + (((2 * c + 1) ^ sw16) << 4)) =
        make_uint4(e2.x, e2.y, e3.x, e3.y);
  }
}

// A quarter of a row (16 int8 -> 32 bytes of the 16-bit tile): narrow tiles are spread over
// all converter threads so that one K block costs one short dependent chain per thread.
template <typename T>
__device__ __forceinline__ void expand_quarter_row(const uint8_t* raw, uint8_t* dst, int r, int c) {
  const uint4 w = *reinterpret_cast<const uint4*>(raw + r * kRow8 + ((c ^ ((r >> 1) & 3)) << 4));
  const uint2 e0 = expand4<T>(w.x), e1 = expand4<T>(w.y), e2 = expand4<T>(w.z), e3 = expand4<T>(w.w);
  uint8_t* dst_row = dst + r * kRow16;
  const int sw16 = r & 7;
  *reinterpret_cast<uint4*>(dst_row + (((2 * c) ^ sw16) << 4)) = make_uint4(e0.x, e0.y, e1.x, e1.y);
  *reinterpret_cast<uint4*>(dst_row + (((2 * c + 1) ^ sw16) << 4)) = make_uint4(e2.x, e2.y, e3.x, e3.y);
}

// ------------------------------------------------------------------------ epilogue
__device__ __forceinline__ float scale_acc(float acc, float s, float b) {
  return __fadd_rn(__fmul_rn(acc, s), b);
}

// Generic path: the 32 fp32 accumulators of columns [c0, c0+32) of this thread's row.
template <typename OutT>
__device__ __forceinline__ void emit_chunk(const KernelParams& p, int tile_a, int tile_b,
                                           int row_in_tile, int c0, const uint32_t (&v)[32]) {
  const int row_a = tile_a * kTileA + row_in_tile;
  const int col_b0 = tile_b * p.bn + c0;
  if (row_a >= p.rows_a || col_b0 >= p.rows_b) return;
  const int N = p.n_channels;
  const OutT* bias = reinterpret_cast<const OutT*>(p.bias);
  OutT* out = reinterpret_cast<OutT*>(p.out);
  if (!p.swap) {
    OutT* dst = out + static_cast<size_t>(row_a) * N + col_b0;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (col_b0 + j < p.rows_b) {
        const float b = bias != nullptr ? to_float<OutT>(bias[col_b0 + j]) : 0.f;
        dst[j] = from_float<OutT>(scale_acc(__uint_as_float(v[j]), __ldg(p.w_scales + col_b0 + j), b));
      }
    }
  } else {
    const float s = __ldg(p.w_scales + row_a);
    const float b = bias != nullptr ? to_float<OutT>(bias[row_a]) : 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int tok = col_b0 + j;
      if (tok < p.rows_b)
        out[static_cast<size_t>(tok) * N + row_a] = from_float<OutT>(scale_acc(__uint_as_float(v[j]), s, b));
    }
  }
}

// Fast path (tokens on rows): convert 32 accumulators and park them in this thread's
// row of the warp's transpose buffer (rows of 128 bytes, 128-byte swizzle).
template <typename OutT, bool HAS_BIAS>
__device__ __forceinline__ void convert_chunk(const KernelParams& p, const float* s_ws, int col0,
                                              int lane, int chunk_half, uint8_t* slab,
                                              const uint32_t (&v)[32]) {
  const OutT* bias = reinterpret_cast<const OutT*>(p.bias);
  uint32_t packed[16];
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 ws = *reinterpret_cast<const float4*>(s_ws + j);
    float2 lo = __fmul2_rn(make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1])),
                           make_float2(ws.x, ws.y));
    float2 hi = __fmul2_rn(make_float2(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])),
                           make_float2(ws.z, ws.w));
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
    const int chunk = chunk_half * 4 + c;
    *reinterpret_cast<uint4*>(slab + lane * 128 + ((chunk ^ sw) << 4)) =
        make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
  }
}

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
    if (row < p.rows_a && col < p.rows_b)
      *reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * p.n_channels + col) = val;
  }
}

}  // namespace
}  // namespace b200q
