// Row-parallel exchange step fused with what follows it in the model: the sum over the
// tensor-parallel ranks (dist.all_reduce(y), nanovllm/layers/linear.py:274-275), the residual add
// and RMSNorm that consume it (nanovllm/layers/layernorm.py:28-40, called from
// nanovllm/models/qwen3.py:160-166) and the per-token int8 quantisation of the next W8A8 layer's
// input (nanovllm/quantization/utils.py:28-32) — in ONE kernel per rank.
//
// Rank r owns token rows [r * M / world, (r + 1) * M / world).  For its rows it
//   1. reads the partial outputs of all ranks (16-byte peer loads over NVLink) and adds them in
//      rank order in fp32, rounding the sum to the 16-bit type: exactly the tensor an all-reduce
//      would have produced (reduce-scatter half);
//   2. adds the residual (kept sharded by rows: each rank only ever needs its own rows),
//      writes the new residual, applies RMSNorm and quantises — the arithmetic and the
//      thread mapping of add_rmsnorm_quant_kernel, so codes and scales are bit-identical to
//      "all-reduce, then b200q_add_rmsnorm_quant_i8";
//   3. writes the int8 codes and the fp32 scale of each row into EVERY rank's input buffer
//      of the next layer (8-byte peer stores, a warp covering whole lines): the all-gather
//      moves one byte per element instead of two.
// Compared with "all-reduce, then norm + quant" a rank receives (world - 1) / world * M * K
// * 3 bytes instead of 4, no 16-bit sum is written to or re-read from memory, and one kernel
// (and one pair of flag barriers) does the work of two.
//
// Flags: the two barriers of the two-shot all-reduce on the same flag pad (shared call
// numbering: calls of the two entry points may be mixed as long as every rank makes the same
// sequence).  Barrier A — every rank's partial output is complete — also guarantees that every
// rank has finished reading the code buffers filled by the previous exchange, so they can be
// overwritten; barrier B — every rank has written its rows everywhere — ends the kernel.
// Every wait is bounded.  Plain loads and stores only.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <climits>
#include <type_traits>

#include "act_quant_device.cuh"
#include "common.h"
#include "peer_sync.cuh"
#include "ptx_sm100.cuh"

namespace b200q {
namespace {

constexpr int kMaxWorld = 8;
// 32-bit slots of a rank's flag pad (the layout of tp_allreduce.cu)
constexpr int kSlotEpoch = 0;
constexpr int kSlotCounter = 1;
constexpr int kSlotA = 16;
constexpr int kSlotB = 32;

struct ExchangeParams {
  const void* partial[kMaxWorld];  // every rank's partial output [M, K]
  unsigned int* pad[kMaxWorld];
  int8_t* xq[kMaxWorld];           // every rank's code buffer [M, K]
  float* scales[kMaxWorld];        // every rank's scale buffer [M]
  const void* residual_in;         // this rank's rows [M / world, K], or nullptr
  void* residual_out;              // this rank's rows, or nullptr
  void* y_out;                     // normalised 16-bit rows of this rank (tests), or nullptr
  const void* weight;              // [K]
  float eps;
  int M, K, rank, world, rows_per_rank;
  int* status;
  long long wait_limit;
  int debug_flags;  // test hook (timing only, results wrong): 64 = codes to the own buffer only,
                    // 128 = read the own partial in place of the peers'
};

template <typename T, int G, int CHUNKS, int W>
__global__ void __launch_bounds__(256)
tp_reduce_norm_quant_kernel(const ExchangeParams p) {
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr int kRowsPerBlock = 256 / G;
  __shared__ unsigned int s_epoch;
  __shared__ int s_flag;  // 0 ok, 1 = a wait gave up, 2 / 3 = this CTA is the rank's last (ok / failed)
  __shared__ float red[8];
  unsigned int* my_pad = p.pad[p.rank];
  if (threadIdx.x == 0) s_flag = 0;
  // launch and set-up overlap the tail of the producing kernel; its output is needed from here
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  __syncthreads();

  // ---- barrier A: every rank's partial output is complete (and its previous reads are over).
  // The `world` flag threads read the call number themselves: one trip to memory less on the
  // path of every CTA than publishing it through shared memory first.
  if (threadIdx.x < p.world) {
    const unsigned int e = *reinterpret_cast<volatile unsigned int*>(my_pad + kSlotEpoch) + 1u;
    if (blockIdx.x == 0) st_release_sys(p.pad[threadIdx.x] + kSlotA + p.rank, e);
    if (!wait_flag(my_pad + kSlotA + threadIdx.x, e, p.wait_limit)) s_flag = 1;
    if (threadIdx.x == 0) s_epoch = e;
  }
  __syncthreads();
  const unsigned int epoch = s_epoch;
  const bool ok = s_flag == 0;

  const int g = threadIdx.x / G, t = threadIdx.x % G;
  const int nchunk = p.K >> 3;
  const T* weight = static_cast<const T*>(p.weight);
  const int row_blocks = (p.rows_per_rank + kRowsPerBlock - 1) / kRowsPerBlock;
  for (int rb = blockIdx.x; ok && rb < row_blocks; rb += gridDim.x) {
    const int local_row = rb * kRowsPerBlock + g;
    const bool active = local_row < p.rows_per_rank;
    const int row = p.rank * p.rows_per_rank + local_row;  // row of the full [M, K] matrices

    // Every load of the row is issued before the first use: CHUNKS x world 16-byte loads per
    // thread in flight, so that a row block costs one trip over NVLink, not one per chunk (the
    // stores below could alias the loads as far as the compiler knows, so it would not hoist
    // them by itself).
    uint4 part[CHUNKS][W];
    uint4 resv_all[CHUNKS];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int idx = c * G + t;
      const bool live = active && idx < nchunk;
      resv_all[c] = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int r = 0; r < W; ++r) {
        part[c][r] = make_uint4(0u, 0u, 0u, 0u);
        if (r < p.world && live)
          part[c][r] = ld_peer16(static_cast<const T*>(p.partial[(p.debug_flags & 128) ? p.rank : r]) +
                                 static_cast<size_t>(row) * p.K + idx * 8);
      }
      if (live && p.residual_in != nullptr)
        resv_all[c] = ld_peer16(static_cast<const T*>(p.residual_in) + static_cast<size_t>(local_row) * p.K + idx * 8);
    }

    float s[CHUNKS][8];
    float sumsq = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int idx = c * G + t;
      const bool live = active && idx < nchunk;
      const uint4 resv = resv_all[c];
      // the all-reduce: fp32 sum in rank order, one rounding to the 16-bit type
      float acc[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
      for (int r = 0; r < W; ++r)
        if (r < p.world) accumulate<kBf16>(acc, part[c][r]);
      const uint4 yv = pack<kBf16>(acc);
      const uint32_t xw[4] = {yv.x, yv.y, yv.z, yv.w};
      const uint32_t rw[4] = {resv.x, resv.y, resv.z, resv.w};
      uint32_t out[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = unpack2<T>(xw[i]), b = unpack2<T>(rw[i]);
        const float s0 = p.residual_in != nullptr ? __fadd_rn(a.x, b.x) : a.x;
        const float s1 = p.residual_in != nullptr ? __fadd_rn(a.y, b.y) : a.y;
        s[c][2 * i] = s0;
        s[c][2 * i + 1] = s1;
        sumsq = __fmaf_rn(s0, s0, sumsq);
        sumsq = __fmaf_rn(s1, s1, sumsq);
        out[i] = pack2<T>(s0, s1);
      }
      if (live && p.residual_out != nullptr)
        *(reinterpret_cast<uint4*>(static_cast<T*>(p.residual_out) + static_cast<size_t>(local_row) * p.K) + idx) =
            make_uint4(out[0], out[1], out[2], out[3]);
    }
    const float total = group_reduce<G, false>(sumsq, red, g);
    const float inv_rms = __frsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(p.K)), p.eps));

    uint4 y[CHUNKS];
    AbsMax2<T> running;
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
        running.add(out[i]);
      }
      y[c] = make_uint4(out[0], out[1], out[2], out[3]);
    }
    const float amax = group_reduce<G, true>(running.value(), red, g);
    if (active) {
      const float scale = fmaxf(__fdiv_rn(amax, 127.0f), 1e-8f);
      const float inv_scale = __frcp_rn(scale);
#pragma unroll
      for (int r = 0; r < W; ++r)
        if (r < p.world && t == r) p.scales[r][row] = scale;  // one lane per destination rank
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int idx = c * G + t;
        if (idx < nchunk) {
          const uint2 q = quant8<T>(y[c], scale, inv_scale);
#pragma unroll
          for (int r = 0; r < W; ++r)
            if (r < p.world && (!(p.debug_flags & 64) || r == p.rank))
              *(reinterpret_cast<uint2*>(p.xq[r] + static_cast<size_t>(row) * p.K) + idx) = q;
          if (p.y_out != nullptr)
            *(reinterpret_cast<uint4*>(static_cast<T*>(p.y_out) + static_cast<size_t>(local_row) * p.K) + idx) = y[c];
        }
      }
    }
  }
  // ---- barrier B: by the last CTA of this rank to get here.  One system-scope release per
  // CTA, folded into the counter update by thread 0 after the CTA barrier (release is
  // cumulative: it also orders the other threads' stores), instead of a fence per thread: with
  // a few hundred CTAs per rank those fences were a visible part of the kernel's fixed cost.
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int done;
    asm volatile("atom.acq_rel.sys.global.add.u32 %0, [%1], 1;"
                 : "=r"(done)
                 : "l"(my_pad + kSlotCounter)
                 : "memory");
    if (done == gridDim.x - 1) {
      my_pad[kSlotCounter] = 0u;
      s_flag = s_flag == 0 ? 2 : 3;
    }
  }
  __syncthreads();
  if (s_flag == 2) {
    if (threadIdx.x < p.world) {
      // the other CTAs' stores were acquired through the counter; the release store keeps
      // them ahead of the flag
      st_release_sys(p.pad[threadIdx.x] + kSlotB + p.rank, epoch);
      if (!wait_flag(my_pad + kSlotB + threadIdx.x, epoch, p.wait_limit)) atomicCAS(p.status, 0, 0x802);
    }
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned int*>(my_pad + kSlotEpoch) = epoch;
  } else if (s_flag != 0 && threadIdx.x == 0) {
    atomicCAS(p.status, 0, 0x801);
    // only the rank's last CTA moves the call count (every CTA reads it at its start)
    if (s_flag == 3) *reinterpret_cast<volatile unsigned int*>(my_pad + kSlotEpoch) = epoch;
  }
}

// One wave: as many CTAs as are resident at once, each walking over its share of the row
// blocks.  (A CTA spends a few microseconds on the opening flag exchange and on its closing
// fence whatever it computes; a second wave would pay those again.)
template <typename T, int G, int CHUNKS, int W>
cudaError_t launch_exchange_g(const ExchangeParams& p, cudaStream_t st) {
  auto kern = tp_reduce_norm_quant_kernel<T, G, CHUNKS, W>;
  static int per_sm[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && per_sm[dev] == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, 256, 0) != cudaSuccess || n < 1) n = 1;
    per_sm[dev] = n;
  }
  const int resident = sm_count() * (dev < 64 ? per_sm[dev] : 1);
  const int row_blocks = (p.rows_per_rank + (256 / G) - 1) / (256 / G);
  const int grid = row_blocks < resident ? row_blocks : resident;
  return launch_overlapped(kern, grid, 256, 0, st, p);
}

template <typename T, int W>
cudaError_t launch_exchange(const ExchangeParams& p, cudaStream_t st) {
  const int K = p.K;
  // same row-group widths as the stand-alone add-RMSNorm quantiser (bit-identical sums)
  if (K <= 32 * 8 * 4) return launch_exchange_g<T, 32, 4, W>(p, st);
  if (K <= 64 * 8 * 4) return launch_exchange_g<T, 64, 4, W>(p, st);
  if (K <= 128 * 8 * 4) return launch_exchange_g<T, 128, 4, W>(p, st);
  if (K <= 256 * 8 * 4) return launch_exchange_g<T, 256, 4, W>(p, st);
  return launch_exchange_g<T, 256, 8, W>(p, st);
}

template <typename T>
cudaError_t launch_exchange_w(const ExchangeParams& p, cudaStream_t st) {
  if (p.world <= 2) return launch_exchange<T, 2>(p, st);
  if (p.world <= 4) return launch_exchange<T, 4>(p, st);
  return launch_exchange<T, 8>(p, st);
}

bool aligned16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; }

}  // namespace
}  // namespace b200q

extern "C" int b200q_tp_reduce_rmsnorm_quant(void* const* peer_partials, void* const* peer_flag_pads,
                                             const void* residual_in, void* residual_out,
                                             const void* weight, float eps, void* const* peer_xq,
                                             void* const* peer_scales, void* y_local, int M, int K,
                                             int rank, int world, int dtype, void* stream) {
  using namespace b200q;
  if (peer_partials == nullptr || peer_flag_pads == nullptr || weight == nullptr ||
      peer_xq == nullptr || peer_scales == nullptr)
    return B200Q_ERR_NULL_POINTER;
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return B200Q_ERR_BAD_ARGUMENT;
  if (dtype != B200Q_DTYPE_F16 && dtype != B200Q_DTYPE_BF16) return B200Q_ERR_BAD_ARGUMENT;
  if (M <= 0 || K <= 0 || static_cast<long long>(M) * K > INT_MAX) return B200Q_ERR_BAD_SHAPE;
  if ((K % 16) != 0 || K > 256 * 8 * 8 || (M % world) != 0) return B200Q_ERR_UNSUPPORTED_SHAPE;
  if (!aligned16(residual_in) || !aligned16(residual_out) || !aligned16(weight) || !aligned16(y_local))
    return B200Q_ERR_MISALIGNED;
  ExchangeParams p{};
  for (int r = 0; r < world; ++r) {
    if (peer_partials[r] == nullptr || peer_flag_pads[r] == nullptr || peer_xq[r] == nullptr ||
        peer_scales[r] == nullptr)
      return B200Q_ERR_NULL_POINTER;
    if (!aligned16(peer_partials[r]) || !aligned16(peer_xq[r]) ||
        (reinterpret_cast<uintptr_t>(peer_scales[r]) & 3u) != 0)
      return B200Q_ERR_MISALIGNED;
    p.partial[r] = peer_partials[r];
    p.pad[r] = static_cast<unsigned int*>(peer_flag_pads[r]);
    p.xq[r] = static_cast<int8_t*>(peer_xq[r]);
    p.scales[r] = static_cast<float*>(peer_scales[r]);
  }
  if (device_cc_major() != 10) return B200Q_ERR_UNSUPPORTED_ARCH;
  p.residual_in = residual_in;
  p.residual_out = residual_out;
  p.y_out = y_local;
  p.weight = weight;
  p.eps = eps;
  p.M = M;
  p.K = K;
  p.rank = rank;
  p.world = world;
  p.rows_per_rank = M / world;
  p.status = device_status_ptr();
  p.wait_limit = peer_wait_limit_cycles();
  p.debug_flags = debug_knob(B200Q_KNOB_FLAGS, 0);
  if (p.status == nullptr) return B200Q_ERR_LAUNCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = dtype == B200Q_DTYPE_BF16 ? launch_exchange_w<__nv_bfloat16>(p, st)
                                            : launch_exchange_w<__half>(p, st);
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch();
  return B200Q_OK;
}
