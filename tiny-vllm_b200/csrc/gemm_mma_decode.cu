// Weight-streaming decode kernels (M <= 64 tokens): split-K inside the CTA, 128-bit int8
// weight loads, in-register dequantisation, warp-level tensor-core MMA.
//
// At decode sizes a linear layer is a stream of the weight matrix past a handful of
// tokens; the cost is launch latency plus one trip to memory, so the kernel is built to
// have EVERY weight byte in flight as early as possible and to finish without a second
// kernel or a global round trip:
//   * a CTA owns 8 output channels and all of K; its 8 warps split K (interleaved blocks
//     of 64), so with N/8 CTAs of 8 warps the whole matrix is requested in one go;
//   * each lane loads 16 contiguous bytes of one weight row per block (4 lanes cover the
//     64-byte block of a channel, 8 channels per warp instruction);
//   * tokens are the M side of mma.sync (m16n8k32 s8 for W8A8, m16n8k16 bf16/f16 for
//     W8A16, weights expanded int8 -> 16 bit in registers, exactly), channels the N side;
//     the K index inside a block is permuted the same way for both operands, which a dot
//     product does not notice, so no shuffles or shared-memory staging are needed;
//   * the 8 partial tiles are summed through shared memory in a fixed order, scaled and
//     stored.
//
// Arithmetic: W8A8  exact int32 sums, then (float(acc) * a_s[m]) * w_s[n] + bias[n]
//                   (nanovllm/quantization/csrc/w8a8_gemm.cu:165-183, 387-390);
//             W8A16 fp32 sums of x * float(q), then acc * s[n] + bias[n]
//                   (nanovllm/quantization/csrc/int8_weight_only_gemm.cu:258-292).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <type_traits>

#include "common.h"
#include "peer_sync.cuh"
#include "ptx_sm100.cuh"

namespace b200q {
namespace {

constexpr int kWarps = 8;          // K split inside the CTA
constexpr int kThreads = kWarps * 32;
constexpr int kChannels = 8;       // output channels per CTA (N side of the MMA)
constexpr int kBlock = 64;         // K elements per block (one 16-byte load per lane)
constexpr int kMaxMT = 4;          // up to 4 token tiles of 16 -> M <= 64

// ---------------------------------------------------------------- fused all-reduce
// Row-parallel layers (nanovllm/layers/linear.py:265-276) sum the ranks' partial results.
// With FUSED kernels that sum happens inside the GEMM kernel, tile by tile, over peer
// memory: CTA c of rank r rounds its partial tile to the output type (exactly what the
// unfused kernel would store) and pushes it into slot r of every OTHER rank's receive area;
// then it collects the same tile of every other rank from its own receive area, adds the
// `world` partials in rank order in fp32 and stores the sum locally.  One NVLink trip, no
// second kernel, and no fence or separate flag on the way: values travel as 8-byte words
// {two 16-bit values, call number}; an aligned 8-byte store arrives whole, so a word whose
// upper half equals the current call number is valid data.  The receiver polls the words
// themselves (bounded).  Receive areas alternate between two halves by call parity, so a
// rank that is one call ahead cannot overwrite words a slower rank still reads; being two
// calls ahead is impossible because finishing a call needs every peer's words of that call.
// Call numbers only grow (0 is skipped on wrap-around; the areas start zero-filled).
struct FuseParams {
  void* recv[8];        // every rank's receive area (both parity halves)
  unsigned int* ctl[8]; // every rank's control words (only the own rank's are used)
  size_t half_bytes;    // bytes of one parity half
  int rank, world;
  long long wait_limit; // SM cycles one wait on a peer may take
};


// part: this CTA's tile in shared memory, [M][8] values of OutT.  All threads call.
template <typename OutT>
__device__ __forceinline__ void exchange_and_sum(const OutT* part, const FuseParams& fp, int M,
                                                 int N, OutT* __restrict__ y, int* status) {
  constexpr bool kBf16 = std::is_same<OutT, __nv_bfloat16>::value;
  constexpr int kWordsPerTok = kChannels / 2;  // 8-byte words of one token row of the tile
  __shared__ unsigned int s_epoch;
  __shared__ int s_fail;
  unsigned int* ctl = fp.ctl[fp.rank];
  if (threadIdx.x == 0) {
    s_epoch = next_epoch(ctl);
    s_fail = 0;
  }
  __syncthreads();  // also publishes `part`
  const unsigned int epoch = s_epoch;
  const size_t half_off = (epoch & 1u) * fp.half_bytes;
  const size_t slot_words = static_cast<size_t>(M) * (N / 2);  // one source rank's partial
  const size_t tile_word0 = static_cast<size_t>(blockIdx.x) * kWordsPerTok;
  const uint32_t* part_w = reinterpret_cast<const uint32_t*>(part);
  const int words = M * kWordsPerTok;

  // push: one 8-byte word {2 values, call number} per (peer, token, channel pair)
  for (int i = threadIdx.x; i < words * fp.world; i += kThreads) {
    const int peer = i / words, wi = i - peer * words;
    if (peer == fp.rank) continue;  // the own tile is taken from shared memory below
    const int tok = wi / kWordsPerTok, pair = wi - tok * kWordsPerTok;
    uint2* dst = reinterpret_cast<uint2*>(static_cast<char*>(fp.recv[peer]) + half_off) +
                 fp.rank * slot_words + static_cast<size_t>(tok) * (N / 2) + tile_word0 + pair;
    st_word8(dst, part_w[wi], epoch);
  }
  // collect and sum in rank order
  const uint2* mine =
      reinterpret_cast<const uint2*>(static_cast<const char*>(fp.recv[fp.rank]) + half_off);
  for (int wi = threadIdx.x; wi < words; wi += kThreads) {
    const int tok = wi / kWordsPerTok, pair = wi - tok * kWordsPerTok;
    const size_t off = static_cast<size_t>(tok) * (N / 2) + tile_word0 + pair;
    float lo = 0.f, hi = 0.f;
    bool ok = true;
    for (int r = 0; r < fp.world; ++r) {
      uint32_t w;
      if (r == fp.rank) {
        w = part_w[wi];
      } else {
        if (!wait_word8(mine + r * slot_words + off, epoch, &w, fp.wait_limit)) ok = false;
      }
      if (kBf16) {
        lo += __uint_as_float(w << 16);
        hi += __uint_as_float(w & 0xFFFF0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
        lo += f.x;
        hi += f.y;
      }
    }
    if (ok) {
      uint32_t out;
      if (kBf16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        out = *reinterpret_cast<const uint32_t*>(&h);
      } else {
        const __half2 h = __floats2half2_rn(lo, hi);
        out = *reinterpret_cast<const uint32_t*>(&h);
      }
      reinterpret_cast<uint32_t*>(y)[static_cast<size_t>(tok) * (N / 2) + tile_word0 + pair] = out;
    } else {
      s_fail = 1;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_fail != 0) atomicCAS(status, 0, 0x601);
    finish_call(ctl, epoch);
  }
}

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

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T>
__device__ __forceinline__ void mma_16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1,
                                                      uint32_t a2, uint32_t a3, uint32_t b0,
                                                      uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16<__half>(float (&c)[4], uint32_t a0, uint32_t a1,
                                               uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four int8 (one word) -> four 16-bit values (two words), exact for all 256 codes.
template <typename T>
__device__ __forceinline__ uint2 expand4(uint32_t w);
template <>
__device__ __forceinline__ uint2 expand4<__half>(uint32_t w) {
  // 0x6400 | u is the half 1024 + u with u = q + 128; subtract 1152
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
  // 0x4B000000 | u is the float 2^23 + u; subtract 2^23 + 128; at most 8 significant bits
  const uint32_t t = w ^ 0x80808080u;
  // packed fp32 adds (each half rounds like the scalar instruction; the sums are exact anyway)
  const float2 m = make_float2(-8388736.f, -8388736.f);
  const float2 f01 = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(t, 0x4B000000u, 0x7540)),
                                            __uint_as_float(__byte_perm(t, 0x4B000000u, 0x7541))), m);
  const float2 f23 = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(t, 0x4B000000u, 0x7542)),
                                            __uint_as_float(__byte_perm(t, 0x4B000000u, 0x7543))), m);
  // the sums are integers of at most 8 significant bits: their bf16 form is the upper half of
  // the fp32 word, taken with a byte permute (the packing conversion runs on a slower pipe)
  return make_uint2(__byte_perm(__float_as_uint(f01.x), __float_as_uint(f01.y), 0x7632),
                    __byte_perm(__float_as_uint(f23.x), __float_as_uint(f23.y), 0x7632));
}

// ------------------------------------------------------------------------- W8A8
// MT = number of 16-token tiles.  Lane (g = lane / 4, t = lane % 4): weight row g of the
// CTA's 8 channels, bytes [16 t, 16 t + 16) of each 64-byte K block; the same byte range
// of token rows g and g + 8 of every token tile.
template <typename OutT, int MT, bool RAW_I32, bool FUSED>
__global__ void __launch_bounds__(kThreads)
w8a8_mma_decode_kernel(const int8_t* __restrict__ xq, const int8_t* __restrict__ w,
                       const float* __restrict__ a_s, const float* __restrict__ w_s,
                       const OutT* __restrict__ bias, void* __restrict__ out, int M, int N, int K,
                       const FuseParams fp, int* status) {
  __shared__ int red[kWarps][MT * 16 * kChannels];
  __shared__ __align__(16) OutT part[FUSED ? MT * 16 * kChannels : 8];
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int ch = blockIdx.x * kChannels + g;
  const bool ch_ok = ch < N;
  const int nblocks = (K + kBlock - 1) / kBlock;
  const int8_t* wrow = w + static_cast<size_t>(ch_ok ? ch : 0) * K + 16 * t;

  int acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[m][i] = 0;

  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (int b0 = warp; b0 < nblocks; b0 += 2 * kWarps) {
    // two K blocks per iteration: both weight loads are issued before any use
    const int b1 = b0 + kWarps;
    const bool ok0 = ch_ok && (b0 * kBlock + 16 * t) < K;
    const bool ok1 = ch_ok && b1 < nblocks && (b1 * kBlock + 16 * t) < K;
    const uint4 w0 = ok0 ? __ldg(reinterpret_cast<const uint4*>(wrow + b0 * kBlock)) : zero;
    const uint4 w1 = ok1 ? __ldg(reinterpret_cast<const uint4*>(wrow + b1 * kBlock)) : zero;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int blk = half == 0 ? b0 : b1;
      if (half == 1 && b1 >= nblocks) break;
      const uint4 wv = half == 0 ? w0 : w1;
      const bool k_ok = (blk * kBlock + 16 * t) < K;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const int r0 = m * 16 + g, r1 = r0 + 8;
        const uint4 x0 = (k_ok && r0 < M)
                             ? __ldg(reinterpret_cast<const uint4*>(
                                   xq + static_cast<size_t>(r0) * K + blk * kBlock + 16 * t))
                             : zero;
        const uint4 x1 = (k_ok && r1 < M)
                             ? __ldg(reinterpret_cast<const uint4*>(
                                   xq + static_cast<size_t>(r1) * K + blk * kBlock + 16 * t))
                             : zero;
        // bytes 0-7 feed the first k32 step (slots 0/1), bytes 8-15 the second
        mma_s8(acc[m], x0.x, x1.x, x0.y, x1.y, wv.x, wv.y);
        mma_s8(acc[m], x0.z, x1.z, x0.w, x1.w, wv.z, wv.w);
      }
    }
  }

  // C fragment: acc[m][0..1] = (token m*16+g, channels 2t, 2t+1), acc[m][2..3] = token + 8
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    int* r = red[warp] + m * 16 * kChannels;
    r[g * kChannels + 2 * t] = acc[m][0];
    r[g * kChannels + 2 * t + 1] = acc[m][1];
    r[(g + 8) * kChannels + 2 * t] = acc[m][2];
    r[(g + 8) * kChannels + 2 * t + 1] = acc[m][3];
  }
  __syncthreads();
  for (int o = threadIdx.x; o < MT * 16 * kChannels; o += kThreads) {
    const int tok = o / kChannels, c = o % kChannels;
    const int n = blockIdx.x * kChannels + c;
    if (tok >= M || n >= N) continue;
    int sum = 0;
#pragma unroll
    for (int wi = 0; wi < kWarps; ++wi) sum += red[wi][o];
    const size_t idx = static_cast<size_t>(tok) * N + n;
    if (RAW_I32) {
      reinterpret_cast<int32_t*>(out)[idx] = sum;
    } else {
      const float b = bias != nullptr ? to_float<OutT>(bias[n]) : 0.f;
      const float v = __fadd_rn(__fmul_rn(__fmul_rn(static_cast<float>(sum), a_s[tok]), w_s[n]), b);
      if (FUSED) {
        part[o] = from_float<OutT>(v);
      } else {
        reinterpret_cast<OutT*>(out)[idx] = from_float<OutT>(v);
      }
    }
  }
  if (FUSED) exchange_and_sum<OutT>(part, fp, M, N, reinterpret_cast<OutT*>(out), status);
}

// ------------------------------------------------------------------------ W8A16
// Same ownership; a 64-element K block is four k16 steps, lane t supplies physical
// k [16 t + 4 j, 16 t + 4 j + 4) to step j (4 weights = one word, 4 activations = 8 bytes).
template <typename T, int MT, bool FUSED>
__global__ void __launch_bounds__(kThreads)
w8a16_mma_decode_kernel(const T* __restrict__ x, const int8_t* __restrict__ w,
                        const float* __restrict__ s, const T* __restrict__ bias,
                        T* __restrict__ y, int M, int N, int K, const FuseParams fp, int* status) {
  __shared__ float red[kWarps][MT * 16 * kChannels];
  __shared__ __align__(16) T part[FUSED ? MT * 16 * kChannels : 8];
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int ch = blockIdx.x * kChannels + g;
  const bool ch_ok = ch < N;
  const int nblocks = (K + kBlock - 1) / kBlock;
  const int8_t* wrow = w + static_cast<size_t>(ch_ok ? ch : 0) * K + 16 * t;

  float acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[m][i] = 0.f;

  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (int b0 = warp; b0 < nblocks; b0 += 2 * kWarps) {
    const int b1 = b0 + kWarps;
    const bool ok0 = ch_ok && (b0 * kBlock + 16 * t) < K;
    const bool ok1 = ch_ok && b1 < nblocks && (b1 * kBlock + 16 * t) < K;
    const uint4 w0 = ok0 ? __ldg(reinterpret_cast<const uint4*>(wrow + b0 * kBlock)) : zero;
    const uint4 w1 = ok1 ? __ldg(reinterpret_cast<const uint4*>(wrow + b1 * kBlock)) : zero;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int blk = half == 0 ? b0 : b1;
      if (half == 1 && b1 >= nblocks) break;
      const uint4 wv = half == 0 ? w0 : w1;
      const bool k_ok = (blk * kBlock + 16 * t) < K;
      const uint2 e0 = expand4<T>(wv.x), e1 = expand4<T>(wv.y), e2 = expand4<T>(wv.z),
                  e3 = expand4<T>(wv.w);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const int r0 = m * 16 + g, r1 = r0 + 8;
        // 16 activations (32 bytes) of each of the two token rows
        const uint4* p0 = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r0) * K +
                                                         blk * kBlock + 16 * t);
        const uint4* p1 = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r1) * K +
                                                         blk * kBlock + 16 * t);
        const bool v0 = k_ok && r0 < M, v1 = k_ok && r1 < M;
        const uint4 x0a = v0 ? __ldg(p0) : zero, x0b = v0 ? __ldg(p0 + 1) : zero;
        const uint4 x1a = v1 ? __ldg(p1) : zero, x1b = v1 ? __ldg(p1 + 1) : zero;
        mma_16<T>(acc[m], x0a.x, x1a.x, x0a.y, x1a.y, e0.x, e0.y);
        mma_16<T>(acc[m], x0a.z, x1a.z, x0a.w, x1a.w, e1.x, e1.y);
        mma_16<T>(acc[m], x0b.x, x1b.x, x0b.y, x1b.y, e2.x, e2.y);
        mma_16<T>(acc[m], x0b.z, x1b.z, x0b.w, x1b.w, e3.x, e3.y);
      }
    }
  }

#pragma unroll
  for (int m = 0; m < MT; ++m) {
    float* r = red[warp] + m * 16 * kChannels;
    r[g * kChannels + 2 * t] = acc[m][0];
    r[g * kChannels + 2 * t + 1] = acc[m][1];
    r[(g + 8) * kChannels + 2 * t] = acc[m][2];
    r[(g + 8) * kChannels + 2 * t + 1] = acc[m][3];
  }
  __syncthreads();
  for (int o = threadIdx.x; o < MT * 16 * kChannels; o += kThreads) {
    const int tok = o / kChannels, c = o % kChannels;
    const int n = blockIdx.x * kChannels + c;
    if (tok >= M || n >= N) continue;
    float sum = 0.f;
#pragma unroll
    for (int wi = 0; wi < kWarps; ++wi) sum = __fadd_rn(sum, red[wi][o]);  // fixed order
    const float b = bias != nullptr ? to_float<T>(bias[n]) : 0.f;
    const T v = from_float<T>(__fadd_rn(__fmul_rn(sum, s[n]), b));
    if (FUSED) {
      part[o] = v;
    } else {
      y[static_cast<size_t>(tok) * N + n] = v;
    }
  }
  if (FUSED) exchange_and_sum<T>(part, fp, M, N, y, status);
}

// (Fused kernels are launched in plain stream order: a kernel that waits for other GPUs
// does not start early.)
// CTAs of a fused kernel wait for the same CTA of the peers, so every CTA of the grid has to
// be resident at once: the launch is refused (the caller then takes the two-kernel route)
// when the grid exceeds what the device holds.
thread_local bool g_fused_refused = false;
thread_local cudaError_t g_launch_error = cudaSuccess;
cudaError_t take_launch_error() {
  cudaError_t e = g_launch_error;
  g_launch_error = cudaSuccess;
  return e != cudaSuccess ? e : cudaGetLastError();
}
template <typename Kernel>
bool all_ctas_resident(Kernel kernel, int grid) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0) != cudaSuccess)
    return false;
  return static_cast<long long>(grid) <= static_cast<long long>(per_sm) * sm_count();
}

template <typename OutT, bool RAW, bool FUSED = false>
void launch_a8(const GemmArgs& a, int mt, const FuseParams& fp = FuseParams{}) {
  const int grid = (a.N + kChannels - 1) / kChannels;
  const int8_t* xq = reinterpret_cast<const int8_t*>(a.x);
  const OutT* bias = reinterpret_cast<const OutT*>(a.bias);
  void* out = RAW ? static_cast<void*>(a.acc_out) : a.y;
#define B200Q_LAUNCH_A8(MT)                                                                  \
  if (FUSED && !all_ctas_resident(w8a8_mma_decode_kernel<OutT, MT, RAW, FUSED>, grid)) {      \
    g_fused_refused = true;                                                                  \
    return;                                                                                  \
  }                                                                                          \
  g_launch_error = launch_maybe_overlapped(                                                  \
      !FUSED, w8a8_mma_decode_kernel<OutT, MT, RAW, FUSED>, grid, kThreads, 0, a.stream, xq,  \
      a.w, a.a_scales, a.w_scales, bias, out, a.M, a.N, a.K, fp, a.status)
  switch (mt) {
    case 1: B200Q_LAUNCH_A8(1); break;
    case 2: B200Q_LAUNCH_A8(2); break;
    case 3: B200Q_LAUNCH_A8(3); break;
    default: B200Q_LAUNCH_A8(4); break;
  }
#undef B200Q_LAUNCH_A8
}

// Plain stream order for the W8A16 decode kernel: back-to-back launches of it ran 5-8 % slower
// when each was allowed to start under its predecessor's tail (measured on chains of 112
// launches at M = 1 and 16), unlike the W8A8 chain, whose small quantiser kernels gain 7-9 %.
template <typename T, bool FUSED = false>
void launch_a16(const GemmArgs& a, int mt, const FuseParams& fp = FuseParams{}) {
  const int grid = (a.N + kChannels - 1) / kChannels;
#define B200Q_LAUNCH_A16(MT)                                                                 \
  if (FUSED && !all_ctas_resident(w8a16_mma_decode_kernel<T, MT, FUSED>, grid)) {             \
    g_fused_refused = true;                                                                  \
    return;                                                                                  \
  }                                                                                          \
  g_launch_error = launch_maybe_overlapped(                                                  \
      false, w8a16_mma_decode_kernel<T, MT, FUSED>, grid, kThreads, 0, a.stream,              \
      reinterpret_cast<const T*>(a.x), a.w, a.w_scales, reinterpret_cast<const T*>(a.bias),   \
      reinterpret_cast<T*>(a.y), a.M, a.N, a.K, fp, a.status)
  switch (mt) {
    case 1: B200Q_LAUNCH_A16(1); break;
    case 2: B200Q_LAUNCH_A16(2); break;
    case 3: B200Q_LAUNCH_A16(3); break;
    default: B200Q_LAUNCH_A16(4); break;
  }
#undef B200Q_LAUNCH_A16
}

}  // namespace

bool mma_decode_applicable(int M) { return M >= 1 && M <= 16 * kMaxMT; }

cudaError_t launch_w8a8_mma_decode(const GemmArgs& a) {
  if (!mma_decode_applicable(a.M)) return cudaErrorInvalidValue;
  const int mt = (a.M + 15) / 16;
  if (a.acc_out != nullptr) {
    launch_a8<__nv_bfloat16, true>(a, mt);
  } else if (a.dtype == B200Q_DTYPE_BF16) {
    launch_a8<__nv_bfloat16, false>(a, mt);
  } else {
    launch_a8<__half, false>(a, mt);
  }
  cudaError_t e = take_launch_error();
  if (e == cudaSuccess) count_launch();
  return e;
}

cudaError_t launch_w8a16_mma_decode(const GemmArgs& a) {
  if (!mma_decode_applicable(a.M)) return cudaErrorInvalidValue;
  const int mt = (a.M + 15) / 16;
  if (a.dtype == B200Q_DTYPE_BF16) {
    launch_a16<__nv_bfloat16>(a, mt);
  } else {
    launch_a16<__half>(a, mt);
  }
  cudaError_t e = take_launch_error();
  if (e == cudaSuccess) count_launch();
  return e;
}

// Fills the exchange parameters; returns a B200Q_* code.
static int make_fuse_params(const GemmArgs& a, void* const* peer_recv, void* const* peer_flags,
                            size_t recv_bytes, int rank, int world, FuseParams* fp) {
  if (peer_recv == nullptr || peer_flags == nullptr) return B200Q_ERR_NULL_POINTER;
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return B200Q_ERR_BAD_ARGUMENT;
  if (a.M > B200Q_FUSED_MAX_M || (a.N % kChannels) != 0) return B200Q_ERR_UNSUPPORTED_SHAPE;
  const size_t half = (recv_bytes / 2) & ~static_cast<size_t>(255);
  // 4 bytes per value on the wire: 16 bits of data and its share of the call number
  if (static_cast<size_t>(world) * a.M * a.N * 4 > half) return B200Q_ERR_WORKSPACE;
  for (int r = 0; r < world; ++r) {
    if (peer_recv[r] == nullptr || peer_flags[r] == nullptr) return B200Q_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(peer_recv[r]) & 255u) != 0 ||
        (reinterpret_cast<uintptr_t>(peer_flags[r]) & 15u) != 0)
      return B200Q_ERR_MISALIGNED;
    fp->recv[r] = peer_recv[r];
    fp->ctl[r] = static_cast<unsigned int*>(peer_flags[r]);
  }
  fp->half_bytes = half;
  fp->rank = rank;
  fp->world = world;
  fp->wait_limit = peer_wait_limit_cycles();
  return B200Q_OK;
}

static int finish_fused_launch() {
  if (g_fused_refused) {
    g_fused_refused = false;
    return B200Q_ERR_UNSUPPORTED_SHAPE;
  }
  cudaError_t e = take_launch_error();
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch();
  return B200Q_OK;
}

int launch_w8a8_mma_decode_fused(const GemmArgs& a, void* const* peer_recv,
                                 void* const* peer_flags, size_t recv_bytes, int rank, int world) {
  FuseParams fp{};
  if (int rc = make_fuse_params(a, peer_recv, peer_flags, recv_bytes, rank, world, &fp)) return rc;
  const int mt = (a.M + 15) / 16;
  if (a.dtype == B200Q_DTYPE_BF16) {
    launch_a8<__nv_bfloat16, false, true>(a, mt, fp);
  } else {
    launch_a8<__half, false, true>(a, mt, fp);
  }
  return finish_fused_launch();
}

int launch_w8a16_mma_decode_fused(const GemmArgs& a, void* const* peer_recv,
                                  void* const* peer_flags, size_t recv_bytes, int rank,
                                  int world) {
  FuseParams fp{};
  if (int rc = make_fuse_params(a, peer_recv, peer_flags, recv_bytes, rank, world, &fp)) return rc;
  const int mt = (a.M + 15) / 16;
  if (a.dtype == B200Q_DTYPE_BF16) {
    launch_a16<__nv_bfloat16, true>(a, mt, fp);
  } else {
    launch_a16<__half, true>(a, mt, fp);
  }
  return finish_fused_launch();
}

}  // namespace b200q
