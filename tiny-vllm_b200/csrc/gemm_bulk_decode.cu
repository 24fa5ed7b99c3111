// Weight-streaming decode kernels for decode-sized batches (M <= 64 tokens) over LARGE weight
// matrices: a persistent grid of one CTA per SM, each CTA owning an equal share of the output
// channels.  Eight lanes of a producer warp each feed one consumer warp through a private ring of
// shared-memory slots filled by TMA (cp.async.bulk.tensor, 128-byte swizzle, completion counted
// on mbarriers); the consumer warps run the same warp-level MMAs as the register-streaming
// kernels of gemm_mma_decode.cu.
//
// Why a second kernel.  The register-streaming kernel gives every 8 output channels a CTA of
// its own; each CTA re-reads the whole activation matrix from L2 (M x K bytes against 8 x K
// bytes of weights: twice the weight stream at M = 16) and has bytes in flight only between
// its start-up and its reduction, so on the 8B model's matrices (25-100 MB) it reaches
// 0.5-0.6 of the copy rate.  Here
//   * an SM asks for its weights through rings that always hold 100-190 KB of requests, none
//     of which occupy registers while they travel, and the first ring-full of weight tiles
//     is requested before the kernel waits for the producer of its activations;
//   * a unit of work is up to 48 channels, so the activations cross L2 -> SM once per 48
//     channels instead of once per 8;
//   * the channels are cut into one equal share per CTA (no 8-row rounding), so every SM
//     streams the same number of bytes and the grid has no tail;
//   * a tile is one TMA instruction per 48 rows x 128 bytes.  (Untiled cp.async.bulk row copies
//     of 0.5-1 KB were tried first: they retire at about one copy per 80 cycles per SM whatever
//     their size, 6-12 bytes per cycle, half of what the register kernel reaches.)
//
// Work split: K is cut into segments of 128 elements; segment s belongs to ring s % 8, which
// one consumer warp reads (or two, each taking half of the tile's rows).  Within a segment lane (g = lane / 4, t = lane % 4) owns elements [32 t, 32 t + 32) of
// weight rows g, g + 8, ..., g + 40 of the unit and of token rows g, g + 8 of every 16-token
// tile.  Which physical k sits in which MMA slot does not matter as long as both operands agree:
// 16-byte piece q of row r lies at r * 128 + ((q ^ (r & 7)) << 4) under the swizzle, and with
// pieces 2 t and 2 t + 1 per lane a quarter warp (two rows, four t) touches all eight 16-byte
// bank groups once.  The eight partial tiles are summed through shared memory in warp order,
// so results do not depend on the launch.
//   W8A8  m16n8k32 s8, exact int32 sums, then (float(acc) * a_s[m]) * w_s[n] + bias[n]
//         (nanovllm/quantization/csrc/w8a8_gemm.cu:165-183, 387-390)
//   W8A16 m16n8k16 f16/bf16 after an exact in-register expansion of the codes, fp32 sums of
//         x * float(q), then acc * s[n] + bias[n]; for at most 8 tokens the channels take the
//         16-row side of the MMA and the tokens the 8-column side (half the MMAs)
//         (nanovllm/quantization/csrc/int8_weight_only_gemm.cu:258-292)
// Rows and columns outside the matrices are zero-filled by TMA, so ragged K needs no masks.
// Every mbarrier wait is bounded; a wait that runs out stops the CTA's loops (the consumer
// warps still meet at their barriers), is reported through the status word, and the producer
// lanes wait, again bounded, for the tiles they still have in flight.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.h"
#include "ptx_sm100.cuh"

namespace b200q {
namespace {

constexpr int kPipes = 8;                        // rings per CTA = producer lanes
// A kernel has kPipes * WPP consumer warps (WPP = warps per ring: 1, or 2 sharing every tile,
// each taking half of its rows) and one producer warp.
constexpr int kSeg = 128;                        // K elements of one segment (one slot)
constexpr int kUnitRows = 48;                    // channels per unit of work (6 MMA n-tiles)
constexpr int kNT = kUnitRows / 8;
constexpr int kMaxSlots = 8;                     // ring depth per consumer warp
constexpr int kMaxMT = 2;  // token tiles: more would not fit the register file beside the prefetch
constexpr int kRedBytes = kPipes * 16 * kUnitRows * 4;
constexpr int kBarBytes = 2 * kPipes * kMaxSlots * 8;
constexpr int kSmemLimit = 227 * 1024;

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
  const uint32_t t = w ^ 0x80808080u;  // 0x6400 | u is the half 1024 + u, u = q + 128
  uint32_t lo = __byte_perm(t, 0x64646464u, 0x4140);
  uint32_t hi = __byte_perm(t, 0x64646464u, 0x4342);
  const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
  const __half2 l = __hsub2(*reinterpret_cast<__half2*>(&lo), bias);
  const __half2 h = __hsub2(*reinterpret_cast<__half2*>(&hi), bias);
  return make_uint2(*reinterpret_cast<const uint32_t*>(&l), *reinterpret_cast<const uint32_t*>(&h));
}
template <>
__device__ __forceinline__ uint2 expand4<__nv_bfloat16>(uint32_t w) {
  const uint32_t t = w ^ 0x80808080u;  // 0x4B000000 | u is the float 2^23 + u
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


// Host-made description of the rings.  Shared memory of a CTA (1 KB aligned):
// [8 rings x slots x weight tile][partial tiles of the consumer warps][full barriers]
// [empty barriers][abort flag].
struct StreamPlan {
  int slots;       // ring depth per consumer warp
  int segs;        // segments of K: ceil(K / 128)
  int unit_rows;   // rows of the weight tile (the largest unit of any CTA), <= 48
  int slot_bytes;  // bytes of a weight tile in shared memory (unit_rows x 128, 1 KB multiple)
  int tx_bytes;    // bytes TMA reports per tile
};

// The CTA's share of the channels, [lo, hi), cut into `units` pieces of at most 48 rows.
struct Share {
  int lo, hi, units;
};
__host__ __device__ __forceinline__ Share share_of(int N, int cta, int ctas) {
  Share s;
  s.lo = static_cast<int>(static_cast<long long>(N) * cta / ctas);
  s.hi = static_cast<int>(static_cast<long long>(N) * (cta + 1) / ctas);
  s.units = (s.hi - s.lo + kUnitRows - 1) / kUnitRows;
  return s;
}
__host__ __device__ __forceinline__ void unit_range(const Share& s, int u, int& ulo, int& rows) {
  const int n = s.hi - s.lo;
  ulo = s.lo + n * u / s.units;
  rows = s.lo + n * (u + 1) / s.units - ulo;
}

template <int THREADS>
__device__ __forceinline__ void consumer_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory");
}

// Producer lane `pipe` (0-7) feeds consumer warp `pipe`: segments pipe, pipe + 8, ... of every
// unit, in order, through that warp's ring.  Weights are constants, so nothing here waits for
// the previous kernel in the stream: the rings fill while that kernel is still finishing.
__device__ __forceinline__ void produce(const CUtensorMap* tm_w, const StreamPlan& p, const Share& sh,
                                        int pipe, uint32_t ring, uint64_t* full, uint64_t* empty,
                                        volatile int* abort_flag) {
  const int my_segs = (p.segs - pipe + kPipes - 1) / kPipes;
  const int total = sh.units * my_segs;
  int it = 0;
  for (; it < total; ++it) {
    const int slot = it % p.slots, use = it / p.slots;
    if (use > 0 &&
        !ptx::mbar_wait(ptx::smem_u32(empty + slot), static_cast<uint32_t>((use - 1) & 1), abort_flag))
      break;
    int ulo, rows;
    unit_range(sh, it / my_segs, ulo, rows);
    const int k0 = (pipe + kPipes * (it % my_segs)) * kSeg;
    const uint32_t bar = ptx::smem_u32(full + slot);
    ptx::mbar_arrive_expect_tx(bar, static_cast<uint32_t>(p.tx_bytes));
    ptx::tma_load_2d(ring + slot * p.slot_bytes, tm_w, bar, k0, ulo);
  }
  if (*abort_flag != 0) {
    // a wait ran out somewhere in the CTA: give the tiles still in flight a bounded time to
    // land before the CTA's shared memory is released
    for (int j = max(0, it - p.slots); j < it; ++j) {
      const uint32_t bar = ptx::smem_u32(full + j % p.slots);
      const uint32_t parity = static_cast<uint32_t>((j / p.slots) & 1);
      for (int tries = 0; tries < (1 << 16) && !ptx::mbar_try_wait(bar, parity); ++tries) {
      }
    }
  }
}

struct CtaSmem {
  uint8_t* base;     // 1 KB aligned
  uint8_t* red;
  uint64_t* full;    // [8][kMaxSlots]
  uint64_t* empty;   // [8][kMaxSlots]
  volatile int* abort_flag;
};
__device__ __forceinline__ CtaSmem carve(uint8_t* raw, const StreamPlan& p) {
  CtaSmem c;
  const uint32_t a = ptx::smem_u32(raw);
  c.base = raw + ((1024u - (a & 1023u)) & 1023u);
  c.red = c.base + kPipes * p.slots * p.slot_bytes;
  c.full = reinterpret_cast<uint64_t*>(c.red + kRedBytes);
  c.empty = c.full + kPipes * kMaxSlots;
  c.abort_flag = reinterpret_cast<volatile int*>(c.empty + kPipes * kMaxSlots);
  return c;
}
__device__ __forceinline__ void init_barriers(const CtaSmem& c, const StreamPlan& p, int wpp) {
  if (threadIdx.x < 2 * kPipes * kMaxSlots) {  // full and empty barriers are adjacent
    // a tile is filled by one TMA load and released by the wpp warps that read it
    ptx::mbar_init(ptx::smem_u32(c.full + threadIdx.x), threadIdx.x < kPipes * kMaxSlots ? 1 : wpp);
    if (threadIdx.x == 0) *c.abort_flag = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();
}

// ------------------------------------------------------------------------- W8A8
// Activations come straight from global memory (they are small and stay in L2): the lane's
// 32 bytes of token rows g and g + 8 of the NEXT segment are requested before the wait for
// the current weight tile, so their latency is covered by a whole segment of work.  (Keeping a
// lane's activations of all its segments in registers for the whole CTA, possible for
// K <= 4096, measured 1-2 us SLOWER: every CTA then asks for the same few lines at once.)
template <typename OutT, int MT, bool RAW_I32, int WPP>
__global__ void __launch_bounds__(kPipes * WPP * 32 + 32, 1)
w8a8_stream_decode_kernel(const __grid_constant__ CUtensorMap tm_w, const int8_t* __restrict__ xq,
                          const float* __restrict__ a_s, const float* __restrict__ w_s,
                          const OutT* __restrict__ bias, void* __restrict__ out, int M, int N, int K,
                          const StreamPlan p, int* status) {
  constexpr int kCW = kPipes * WPP, kCT = kCW * 32;  // consumer warps / threads
  constexpr int NTW = kNT / WPP;                     // 8-row MMA tiles per consumer warp
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const CtaSmem sm = carve(smem_raw, p);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Share sh = share_of(N, blockIdx.x, gridDim.x);
  if (threadIdx.x == kCT) ptx::tma_prefetch_desc(&tm_w);
  init_barriers(sm, p, WPP);
  ptx::grid_launch_dependents();
  if (warp == kCW) {
    if (lane < kPipes)
      produce(&tm_w, p, sh, lane, ptx::smem_u32(sm.base) + lane * p.slots * p.slot_bytes,
              sm.full + lane * kMaxSlots, sm.empty + lane * kMaxSlots, sm.abort_flag);
    return;
  }
  ptx::grid_dependency_wait();  // activations and their scales come from the previous kernel

  const int g = lane >> 2, t = lane & 3;
  const int pipe = warp % kPipes, part = warp / kPipes;  // part: which NTW tiles of the unit
  const uint8_t* ring = sm.base + pipe * p.slots * p.slot_bytes;
  uint64_t* full = sm.full + pipe * kMaxSlots;
  uint64_t* empty = sm.empty + pipe * kMaxSlots;
  int* red = reinterpret_cast<int*>(sm.red);
  // swizzled positions of this lane's two 16-byte pieces in a 128-byte row whose index is g mod 8
  const int o0 = g * 128 + (((2 * t) ^ g) << 4), o1 = g * 128 + (((2 * t + 1) ^ g) << 4);
  const int my_segs = (p.segs - pipe + kPipes - 1) / kPipes;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  // x[m][0..1] = pieces of token row m*16+g, x[m][2..3] = of token row m*16+g+8
  auto load_x = [&](int c, uint4 (&x)[MT][4]) {
    const int k = (pipe + kPipes * c) * kSeg + 32 * t;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const int r0 = m * 16 + g, r1 = r0 + 8;
      const int8_t* p0 = xq + static_cast<size_t>(r0) * K + k;
      const int8_t* p1 = xq + static_cast<size_t>(r1) * K + k;
      x[m][0] = (r0 < M && k < K) ? __ldg(reinterpret_cast<const uint4*>(p0)) : zero;
      x[m][1] = (r0 < M && k + 16 < K) ? __ldg(reinterpret_cast<const uint4*>(p0 + 16)) : zero;
      x[m][2] = (r1 < M && k < K) ? __ldg(reinterpret_cast<const uint4*>(p1)) : zero;
      x[m][3] = (r1 < M && k + 16 < K) ? __ldg(reinterpret_cast<const uint4*>(p1 + 16)) : zero;
    }
  };

  uint4 xc[MT][4], xn[MT][4];
  if (sh.units > 0 && my_segs > 0) load_x(0, xc);
  bool alive = true;
  int it = 0;
  for (int u = 0; u < sh.units; ++u) {
    int ulo, rows;
    unit_range(sh, u, ulo, rows);
    int acc[MT][NTW][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int j = 0; j < NTW; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m][j][i] = 0;

    auto segment = [&](const uint4 (&xv)[MT][4]) {
      const int slot = it % p.slots;
      if (alive)
        alive = ptx::mbar_wait(ptx::smem_u32(full + slot), static_cast<uint32_t>((it / p.slots) & 1),
                               sm.abort_flag);
      if (alive) {
        const uint8_t* ws = ring + slot * p.slot_bytes;
#pragma unroll
        for (int j = 0; j < NTW; ++j) {
          const int jj = part * NTW + j;  // tile of the unit
          if (jj * 8 < rows) {
            const uint4 w0 = *reinterpret_cast<const uint4*>(ws + jj * 1024 + o0);
            const uint4 w1 = *reinterpret_cast<const uint4*>(ws + jj * 1024 + o1);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              // each pair of words is one k32 step: slots 4t..4t+3 and 16+4t..16+4t+3
              mma_s8(acc[m][j], xv[m][0].x, xv[m][2].x, xv[m][0].y, xv[m][2].y, w0.x, w0.y);
              mma_s8(acc[m][j], xv[m][0].z, xv[m][2].z, xv[m][0].w, xv[m][2].w, w0.z, w0.w);
              mma_s8(acc[m][j], xv[m][1].x, xv[m][3].x, xv[m][1].y, xv[m][3].y, w1.x, w1.y);
              mma_s8(acc[m][j], xv[m][1].z, xv[m][3].z, xv[m][1].w, xv[m][3].w, w1.z, w1.w);
            }
          }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(empty + slot));
      }
      ++it;
    };
    for (int c = 0; c < my_segs; ++c) {
      if (c + 1 < my_segs || u + 1 < sh.units) load_x(c + 1 < my_segs ? c + 1 : 0, xn);
      segment(xc);
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int i = 0; i < 4; ++i) xc[m][i] = xn[m][i];
    }

    // C fragment: acc[m][j][0..1] = (token m*16+g, channels 8j+2t, +1), [2..3] = token + 8
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      int* r = red + pipe * (16 * kUnitRows) + part * NTW * 8;
#pragma unroll
      for (int j = 0; j < NTW; ++j) {
        r[g * kUnitRows + j * 8 + 2 * t] = acc[m][j][0];
        r[g * kUnitRows + j * 8 + 2 * t + 1] = acc[m][j][1];
        r[(g + 8) * kUnitRows + j * 8 + 2 * t] = acc[m][j][2];
        r[(g + 8) * kUnitRows + j * 8 + 2 * t + 1] = acc[m][j][3];
      }
      consumer_barrier<kCT>();
      for (int o = threadIdx.x; o < 16 * kUnitRows; o += kCT) {
        const int tok = m * 16 + o / kUnitRows, ch = o % kUnitRows;
        if (tok >= M || ch >= rows) continue;
        int sum = 0;
#pragma unroll
        for (int wi = 0; wi < kPipes; ++wi) sum += red[wi * (16 * kUnitRows) + o];
        const int n = ulo + ch;
        const size_t idx = static_cast<size_t>(tok) * N + n;
        if (RAW_I32) {
          reinterpret_cast<int32_t*>(out)[idx] = sum;
        } else {
          const float b = bias != nullptr ? to_float<OutT>(bias[n]) : 0.f;
          const float v =
              __fadd_rn(__fmul_rn(__fmul_rn(static_cast<float>(sum), a_s[tok]), w_s[n]), b);
          reinterpret_cast<OutT*>(out)[idx] = from_float<OutT>(v);
        }
      }
      consumer_barrier<kCT>();
    }
  }
  if (threadIdx.x == 0 && *sm.abort_flag != 0)
    atomicCAS(status, 0, 0x900 | (static_cast<int>(blockIdx.x) << 12));
}

// ------------------------------------------------------------------------ W8A16
// The lane's 32 activations of a segment are 64 contiguous bytes per token row.  Weight word i
// of the lane (4 codes) meets activation words 2 i and 2 i + 1 (2 values each) in one k16 step.
template <typename T, int MT, int WPP>
__global__ void __launch_bounds__(kPipes * WPP * 32 + 32, 1)
w8a16_stream_decode_kernel(const __grid_constant__ CUtensorMap tm_w, const T* __restrict__ x,
                           const float* __restrict__ sc, const T* __restrict__ bias,
                           T* __restrict__ y, int M, int N, int K, const StreamPlan p, int* status) {
  constexpr int kCW = kPipes * WPP, kCT = kCW * 32;  // consumer warps / threads
  constexpr int NTW = kNT / WPP;                     // 8-row MMA tiles per consumer warp
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const CtaSmem sm = carve(smem_raw, p);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Share sh = share_of(N, blockIdx.x, gridDim.x);
  if (threadIdx.x == kCT) ptx::tma_prefetch_desc(&tm_w);
  init_barriers(sm, p, WPP);
  ptx::grid_launch_dependents();
  if (warp == kCW) {
    if (lane < kPipes)
      produce(&tm_w, p, sh, lane, ptx::smem_u32(sm.base) + lane * p.slots * p.slot_bytes,
              sm.full + lane * kMaxSlots, sm.empty + lane * kMaxSlots, sm.abort_flag);
    return;
  }
  ptx::grid_dependency_wait();  // activations come from the previous kernel in the stream

  const int g = lane >> 2, t = lane & 3;
  const int pipe = warp % kPipes, part = warp / kPipes;  // part: which NTW tiles of the unit
  const uint8_t* ring = sm.base + pipe * p.slots * p.slot_bytes;
  uint64_t* full = sm.full + pipe * kMaxSlots;
  uint64_t* empty = sm.empty + pipe * kMaxSlots;
  float* red = reinterpret_cast<float*>(sm.red);
  const int o0 = g * 128 + (((2 * t) ^ g) << 4), o1 = g * 128 + (((2 * t + 1) ^ g) << 4);
  const int my_segs = (p.segs - pipe + kPipes - 1) / kPipes;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  // xa[m][0..3] = the 32 values of token row m*16+g, xb[m][0..3] = of token row m*16+g+8
  auto load_x = [&](int c, uint4 (&xa)[MT][4], uint4 (&xb)[MT][4]) {
    const int k = (pipe + kPipes * c) * kSeg + 32 * t;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const int r0 = m * 16 + g, r1 = r0 + 8;
      const T* p0 = x + static_cast<size_t>(r0) * K + k;
      const T* p1 = x + static_cast<size_t>(r1) * K + k;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bool k_ok = k + 8 * j < K;  // K is a multiple of 16: a piece is inside or outside
        xa[m][j] = (r0 < M && k_ok) ? __ldg(reinterpret_cast<const uint4*>(p0) + j) : zero;
        xb[m][j] = (r1 < M && k_ok) ? __ldg(reinterpret_cast<const uint4*>(p1) + j) : zero;
      }
    }
  };

  uint4 ca[MT][4], cb[MT][4], na[MT][4], nb[MT][4];
  if (sh.units > 0 && my_segs > 0) load_x(0, ca, cb);
  bool alive = true;
  int it = 0;
  for (int u = 0; u < sh.units; ++u) {
    int ulo, rows;
    unit_range(sh, u, ulo, rows);
    float acc[MT][NTW][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int j = 0; j < NTW; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m][j][i] = 0.f;

    for (int c = 0; c < my_segs; ++c, ++it) {
      if (c + 1 < my_segs || u + 1 < sh.units) load_x(c + 1 < my_segs ? c + 1 : 0, na, nb);
      const int slot = it % p.slots;
      if (alive)
        alive = ptx::mbar_wait(ptx::smem_u32(full + slot), static_cast<uint32_t>((it / p.slots) & 1),
                               sm.abort_flag);
      if (alive) {
        const uint8_t* ws = ring + slot * p.slot_bytes;
#pragma unroll
        for (int j = 0; j < NTW; ++j) {
          const int jj = part * NTW + j;  // tile of the unit
          if (jj * 8 < rows) {
            const uint4 w0 = *reinterpret_cast<const uint4*>(ws + jj * 1024 + o0);
            const uint4 w1 = *reinterpret_cast<const uint4*>(ws + jj * 1024 + o1);
            const uint2 e0 = expand4<T>(w0.x), e1 = expand4<T>(w0.y), e2 = expand4<T>(w0.z),
                        e3 = expand4<T>(w0.w), e4 = expand4<T>(w1.x), e5 = expand4<T>(w1.y),
                        e6 = expand4<T>(w1.z), e7 = expand4<T>(w1.w);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              mma_16<T>(acc[m][j], ca[m][0].x, cb[m][0].x, ca[m][0].y, cb[m][0].y, e0.x, e0.y);
              mma_16<T>(acc[m][j], ca[m][0].z, cb[m][0].z, ca[m][0].w, cb[m][0].w, e1.x, e1.y);
              mma_16<T>(acc[m][j], ca[m][1].x, cb[m][1].x, ca[m][1].y, cb[m][1].y, e2.x, e2.y);
              mma_16<T>(acc[m][j], ca[m][1].z, cb[m][1].z, ca[m][1].w, cb[m][1].w, e3.x, e3.y);
              mma_16<T>(acc[m][j], ca[m][2].x, cb[m][2].x, ca[m][2].y, cb[m][2].y, e4.x, e4.y);
              mma_16<T>(acc[m][j], ca[m][2].z, cb[m][2].z, ca[m][2].w, cb[m][2].w, e5.x, e5.y);
              mma_16<T>(acc[m][j], ca[m][3].x, cb[m][3].x, ca[m][3].y, cb[m][3].y, e6.x, e6.y);
              mma_16<T>(acc[m][j], ca[m][3].z, cb[m][3].z, ca[m][3].w, cb[m][3].w, e7.x, e7.y);
            }
          }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(empty + slot));
      }
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ca[m][i] = na[m][i];
          cb[m][i] = nb[m][i];
        }
    }

#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float* r = red + pipe * (16 * kUnitRows) + part * NTW * 8;
#pragma unroll
      for (int j = 0; j < NTW; ++j) {
        r[g * kUnitRows + j * 8 + 2 * t] = acc[m][j][0];
        r[g * kUnitRows + j * 8 + 2 * t + 1] = acc[m][j][1];
        r[(g + 8) * kUnitRows + j * 8 + 2 * t] = acc[m][j][2];
        r[(g + 8) * kUnitRows + j * 8 + 2 * t + 1] = acc[m][j][3];
      }
      consumer_barrier<kCT>();
      for (int o = threadIdx.x; o < 16 * kUnitRows; o += kCT) {
        const int tok = m * 16 + o / kUnitRows, ch = o % kUnitRows;
        if (tok >= M || ch >= rows) continue;
        float sum = 0.f;
#pragma unroll
        for (int wi = 0; wi < kPipes; ++wi)
          sum = __fadd_rn(sum, red[wi * (16 * kUnitRows) + o]);  // fixed order
        const int n = ulo + ch;
        const float b = bias != nullptr ? to_float<T>(bias[n]) : 0.f;
        y[static_cast<size_t>(tok) * N + n] = from_float<T>(__fadd_rn(__fmul_rn(sum, sc[n]), b));
      }
      consumer_barrier<kCT>();
    }
  }
  if (threadIdx.x == 0 && *sm.abort_flag != 0)
    atomicCAS(status, 0, 0x900 | (static_cast<int>(blockIdx.x) << 12));
}

// ------------------------------------------------- W8A16, at most 8 tokens
// With 8 tokens or fewer the CHANNELS go on the 16-row side of the MMA and the tokens on its
// 8-column side: one m16n8k16 covers 16 channels (rows g and g + 8 of a pair of 8-row tiles),
// so a segment costs 24 MMAs instead of 48, and a lane loads one token row (g) instead of two.
// WPP = 2 (not instantiated: measured no faster) would let two consumer warps per ring split the
// lane's eight weight words of a segment, the first and the second 16-byte piece with the
// matching halves of the activations.  Everything else — rings, producer, expansion,
// fixed-order reduction — is as above.
template <typename T, int WPP>
__global__ void __launch_bounds__(kPipes * WPP * 32 + 32, 1)
w8a16_stream_decode_m8_kernel(const __grid_constant__ CUtensorMap tm_w, const T* __restrict__ x,
                              const float* __restrict__ sc, const T* __restrict__ bias,
                              T* __restrict__ y, int M, int N, int K, const StreamPlan p,
                              int* status) {
  constexpr int kCW = kPipes * WPP, kCT = kCW * 32;
  constexpr int kMT16 = kNT / 2;   // 16-channel MMA tiles per unit
  constexpr int kHalves = 2 / WPP; // 16-byte weight pieces per lane and warp
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const CtaSmem sm = carve(smem_raw, p);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Share sh = share_of(N, blockIdx.x, gridDim.x);
  if (threadIdx.x == kCT) ptx::tma_prefetch_desc(&tm_w);
  init_barriers(sm, p, WPP);
  ptx::grid_launch_dependents();
  if (warp == kCW) {
    if (lane < kPipes)
      produce(&tm_w, p, sh, lane, ptx::smem_u32(sm.base) + lane * p.slots * p.slot_bytes,
              sm.full + lane * kMaxSlots, sm.empty + lane * kMaxSlots, sm.abort_flag);
    return;
  }
  ptx::grid_dependency_wait();  // activations come from the previous kernel in the stream

  const int g = lane >> 2, t = lane & 3;
  const int pipe = warp % kPipes, part = warp / kPipes;  // part: which piece (WPP = 2)
  const uint8_t* ring = sm.base + pipe * p.slots * p.slot_bytes;
  uint64_t* full = sm.full + pipe * kMaxSlots;
  uint64_t* empty = sm.empty + pipe * kMaxSlots;
  float* red = reinterpret_cast<float*>(sm.red);
  // swizzled position of the lane's piece(s): piece 2 t + h of a row whose index is g mod 8
  int off[kHalves];
#pragma unroll
  for (int h = 0; h < kHalves; ++h)
    off[h] = g * 128 + (((2 * t + (WPP == 2 ? part : h)) ^ g) << 4);
  const int my_segs = (p.segs - pipe + kPipes - 1) / kPipes;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  // token row g: the 16 values that meet piece h are activation pieces 2 h and 2 h + 1
  auto load_x = [&](int c, uint4 (&xv)[2 * kHalves]) {
    const int k = (pipe + kPipes * c) * kSeg + 32 * t + (WPP == 2 ? 16 * part : 0);
    const T* p0 = x + static_cast<size_t>(g) * K + k;
#pragma unroll
    for (int j = 0; j < 2 * kHalves; ++j)
      xv[j] = (g < M && k + 8 * j < K) ? __ldg(reinterpret_cast<const uint4*>(p0) + j) : zero;
  };

  uint4 xc[2 * kHalves], xn[2 * kHalves];
  if (sh.units > 0 && my_segs > 0) load_x(0, xc);
  bool alive = true;
  int it = 0;
  for (int u = 0; u < sh.units; ++u) {
    int ulo, rows;
    unit_range(sh, u, ulo, rows);
    float acc[kMT16][4];
#pragma unroll
    for (int q = 0; q < kMT16; ++q)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[q][i] = 0.f;

    for (int c = 0; c < my_segs; ++c, ++it) {
      if (c + 1 < my_segs || u + 1 < sh.units) load_x(c + 1 < my_segs ? c + 1 : 0, xn);
      const int slot = it % p.slots;
      if (alive)
        alive = ptx::mbar_wait(ptx::smem_u32(full + slot), static_cast<uint32_t>((it / p.slots) & 1),
                               sm.abort_flag);
      if (alive) {
        const uint8_t* ws = ring + slot * p.slot_bytes;
#pragma unroll
        for (int q = 0; q < kMT16; ++q) {
          if (q * 16 < rows) {
#pragma unroll
            for (int h = 0; h < kHalves; ++h) {
              // channel 16 q + g (tile 2 q) and channel 16 q + 8 + g (tile 2 q + 1)
              const uint4 a = *reinterpret_cast<const uint4*>(ws + (2 * q) * 1024 + off[h]);
              const uint4 b = *reinterpret_cast<const uint4*>(ws + (2 * q + 1) * 1024 + off[h]);
              const uint4 x0 = xc[2 * h], x1 = xc[2 * h + 1];
              uint2 ea, eb;
              // weight word i of the piece meets activation words 2 i and 2 i + 1
              ea = expand4<T>(a.x); eb = expand4<T>(b.x);
              mma_16<T>(acc[q], ea.x, eb.x, ea.y, eb.y, x0.x, x0.y);
              ea = expand4<T>(a.y); eb = expand4<T>(b.y);
              mma_16<T>(acc[q], ea.x, eb.x, ea.y, eb.y, x0.z, x0.w);
              ea = expand4<T>(a.z); eb = expand4<T>(b.z);
              mma_16<T>(acc[q], ea.x, eb.x, ea.y, eb.y, x1.x, x1.y);
              ea = expand4<T>(a.w); eb = expand4<T>(b.w);
              mma_16<T>(acc[q], ea.x, eb.x, ea.y, eb.y, x1.z, x1.w);
            }
          }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(empty + slot));
      }
#pragma unroll
      for (int i = 0; i < 2 * kHalves; ++i) xc[i] = xn[i];
    }

    // C fragment: acc[q][0..1] = (channel 16q+g, tokens 2t, 2t+1), [2..3] = channel 16q+8+g.
    // One partial tile [8 tokens][48 channels] per consumer warp.
    float* r = red + warp * (8 * kUnitRows);
#pragma unroll
    for (int q = 0; q < kMT16; ++q) {
      r[(2 * t) * kUnitRows + 16 * q + g] = acc[q][0];
      r[(2 * t + 1) * kUnitRows + 16 * q + g] = acc[q][1];
      r[(2 * t) * kUnitRows + 16 * q + 8 + g] = acc[q][2];
      r[(2 * t + 1) * kUnitRows + 16 * q + 8 + g] = acc[q][3];
    }
    consumer_barrier<kCT>();
    for (int o = threadIdx.x; o < 8 * kUnitRows; o += kCT) {
      const int tok = o / kUnitRows, ch = o % kUnitRows;
      if (tok >= M || ch >= rows) continue;
      float sum = 0.f;
#pragma unroll
      for (int wi = 0; wi < kCW; ++wi)
        sum = __fadd_rn(sum, red[wi * (8 * kUnitRows) + o]);  // fixed order
      const int n = ulo + ch;
      const float b = bias != nullptr ? to_float<T>(bias[n]) : 0.f;
      y[static_cast<size_t>(tok) * N + n] = from_float<T>(__fadd_rn(__fmul_rn(sum, sc[n]), b));
    }
    consumer_barrier<kCT>();
  }
  if (threadIdx.x == 0 && *sm.abort_flag != 0)
    atomicCAS(status, 0, 0x900 | (static_cast<int>(blockIdx.x) << 12));
}

// ------------------------------------------------------------------------ host
int grid_for(int N) { return N < sm_count() ? N : sm_count(); }

bool make_plan(int M, int N, int K, bool a16, StreamPlan& p) {
  const int grid = grid_for(N);
  // the largest unit of any CTA: shares differ by at most one row, units of a share too
  const int share = (N + grid - 1) / grid;
  const int units = (share + kUnitRows - 1) / kUnitRows;
  p.unit_rows = (share + units - 1) / units;
  p.slot_bytes = (p.unit_rows * 128 + 1023) / 1024 * 1024;
  p.tx_bytes = p.unit_rows * 128;
  p.segs = (K + kSeg - 1) / kSeg;
  const int fixed = kRedBytes + kBarBytes + 16 + 1024;  // + slack for the 1 KB alignment
  p.slots = (kSmemLimit - fixed) / (kPipes * p.slot_bytes);
  if (p.slots > kMaxSlots) p.slots = kMaxSlots;
  const int want = debug_knob(B200Q_KNOB_BULK_SLOTS, 0);  // tuning: a shallower ring
  if (want >= 2 && want < p.slots) p.slots = want;
  (void)M;
  (void)a16;
  return p.slots >= 2;
}

size_t plan_smem(const StreamPlan& p) {
  return static_cast<size_t>(kPipes) * p.slots * p.slot_bytes + kRedBytes + kBarBytes + 16 + 1024;
}

// The kernel is a template ARGUMENT, so every kernel has a flag of its own (kernels of one
// signature share a function-pointer type).
template <auto kernel, typename... Args>
cudaError_t launch_stream(int grid, int threads, size_t smem, cudaStream_t stream, Args... args) {
  static bool raised[64] = {false};  // per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !raised[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return e;
    if (dev < 64) raised[dev] = true;
  }
  return launch_overlapped(kernel, dim3(grid), dim3(threads), smem, stream, args...);
}

}  // namespace

// Decode-sized batches over matrices large enough that every SM gets a share worth a ring.
// Thresholds from graph-replayed launches of the Qwen3-0.6B and -8B projections and the 8B
// model's 8-way shards: below 6-8 MB the register-streaming kernels (one short CTA per 8
// channels) are as fast or faster.  Knob BULK_DECODE: 1 = never, 2 = wherever the kernel can run.
bool bulk_decode_applicable(int M, int N, int K, bool a16) {
  const int knob = debug_knob(B200Q_KNOB_BULK_DECODE, 0);
  if (knob == 1) return false;
  // 16-bit activations: one token tile (two tiles plus their prefetch exceed the register file)
  if (M < 1 || M > (a16 ? 16 : 16 * kMaxMT) || K < 16 || (K % 16) != 0 || N < 1) return false;
  StreamPlan p;
  if (!make_plan(M, N, K, a16, p)) return false;
  if (knob == 2) return true;
  return static_cast<long long>(N) * K >= ((a16 ? 6ll : 8ll) << 20) && N >= 8 * sm_count();
}

cudaError_t launch_w8a8_bulk_decode(const GemmArgs& a) {
  StreamPlan p;
  if (!make_plan(a.M, a.N, a.K, false, p)) return cudaErrorInvalidValue;
  CUtensorMap tm_w;
  if (!get_tensor_map(a.w, a.N, a.K, p.unit_rows, 128, &tm_w)) return cudaErrorInvalidValue;
  const int8_t* xq = reinterpret_cast<const int8_t*>(a.x);
  const int grid = grid_for(a.N);
  const size_t smem = plan_smem(p);
  cudaError_t e = cudaSuccess;
#define B200Q_STREAM_A8(MT, WPP)                                                                   \
  if (a.acc_out != nullptr)                                                                        \
    e = launch_stream<w8a8_stream_decode_kernel<__nv_bfloat16, MT, true, WPP>>(                     \
        grid, kPipes * WPP * 32 + 32, smem, a.stream, tm_w, xq, a.a_scales, a.w_scales,             \
        static_cast<const __nv_bfloat16*>(nullptr), static_cast<void*>(a.acc_out), a.M, a.N, a.K,   \
        p, a.status);                                                                               \
  else if (a.dtype == B200Q_DTYPE_BF16)                                                            \
    e = launch_stream<w8a8_stream_decode_kernel<__nv_bfloat16, MT, false, WPP>>(                    \
        grid, kPipes * WPP * 32 + 32, smem, a.stream, tm_w, xq, a.a_scales, a.w_scales,             \
        static_cast<const __nv_bfloat16*>(a.bias), a.y, a.M, a.N, a.K, p, a.status);                \
  else                                                                                             \
    e = launch_stream<w8a8_stream_decode_kernel<__half, MT, false, WPP>>(                           \
        grid, kPipes * WPP * 32 + 32, smem, a.stream, tm_w, xq, a.a_scales, a.w_scales,             \
        static_cast<const __half*>(a.bias), a.y, a.M, a.N, a.K, p, a.status)
  // One token tile: two consumer warps per ring (more warps to cover the latencies of the
  // ring waits and the activation loads: 3-9 % on the 8B projections).  Two token tiles do not
  // fit the register file of 17 warps without spilling (M = 32: 28 against 17.6 us).
  if (a.M <= 16 && debug_knob(B200Q_KNOB_BULK_WPP, 2) == 2) {
    B200Q_STREAM_A8(1, 2);
  } else if (a.M <= 16) {
    B200Q_STREAM_A8(1, 1);
  } else {
    B200Q_STREAM_A8(2, 1);
  }
#undef B200Q_STREAM_A8
  if (e == cudaSuccess) count_launch();
  return e;
}

cudaError_t launch_w8a16_bulk_decode(const GemmArgs& a) {
  StreamPlan p;
  if (!make_plan(a.M, a.N, a.K, true, p)) return cudaErrorInvalidValue;
  CUtensorMap tm_w;
  if (!get_tensor_map(a.w, a.N, a.K, p.unit_rows, 128, &tm_w)) return cudaErrorInvalidValue;
  const int grid = grid_for(a.N);
  const size_t smem = plan_smem(p);
  cudaError_t e = cudaSuccess;
#define B200Q_STREAM_A16(MT, WPP)                                                                  \
  if (a.dtype == B200Q_DTYPE_BF16)                                                                 \
    e = launch_stream<w8a16_stream_decode_kernel<__nv_bfloat16, MT, WPP>>(                          \
        grid, kPipes * WPP * 32 + 32, smem, a.stream, tm_w, static_cast<const __nv_bfloat16*>(a.x), \
        a.w_scales, static_cast<const __nv_bfloat16*>(a.bias), static_cast<__nv_bfloat16*>(a.y),    \
        a.M, a.N, a.K, p, a.status);                                                                \
  else                                                                                             \
    e = launch_stream<w8a16_stream_decode_kernel<__half, MT, WPP>>(                                 \
        grid, kPipes * WPP * 32 + 32, smem, a.stream, tm_w, static_cast<const __half*>(a.x),        \
        a.w_scales, static_cast<const __half*>(a.bias), static_cast<__half*>(a.y), a.M, a.N, a.K,   \
        p, a.status)
  // one consumer warp per ring: with two, each pair loads the activations twice and the 16-bit
  // fragments spill (gate_up at M = 1: 37.5 against 34.2 us)
  // knob BULK_WPP = 1: the 16-token kernel also for M <= 8 (tests compare the two forms)
  if (a.M <= 8 && debug_knob(B200Q_KNOB_BULK_WPP, 0) != 1) {
    // one warp per ring: splitting the lane's eight words between two warps (the template's
    // WPP = 2) measured the same (26.95 against 27.11 us on gate_up)
    if (a.dtype == B200Q_DTYPE_BF16)
      e = launch_stream<w8a16_stream_decode_m8_kernel<__nv_bfloat16, 1>>(
          grid, kPipes * 32 + 32, smem, a.stream, tm_w, static_cast<const __nv_bfloat16*>(a.x), a.w_scales,
          static_cast<const __nv_bfloat16*>(a.bias), static_cast<__nv_bfloat16*>(a.y), a.M, a.N, a.K, p,
          a.status);
    else
      e = launch_stream<w8a16_stream_decode_m8_kernel<__half, 1>>(
          grid, kPipes * 32 + 32, smem, a.stream, tm_w, static_cast<const __half*>(a.x), a.w_scales,
          static_cast<const __half*>(a.bias), static_cast<__half*>(a.y), a.M, a.N, a.K, p, a.status);
  } else {
    B200Q_STREAM_A16(1, 1);
  }
#undef B200Q_STREAM_A16
  if (e == cudaSuccess) count_launch();
  return e;
}

}  // namespace b200q
