// Sum all-reduce of a 16-bit tensor across the tensor-parallel ranks of one node, over
// peer memory (NVLink / NVSwitch), in place — the exchange step after a row-parallel
// linear (reference: dist.all_reduce(y) at nanovllm/layers/linear.py:274-275).
//
// Every rank passes the device addresses of all ranks' buffers (symmetric allocation:
// same size, mapped into every process) and of all ranks' flag pads.  Two-shot scheme:
//   1. flag barrier A: "my partial result is complete" (guaranteed by stream order on the
//      sender, announced by one release store per peer);
//   2. rank r sums chunk range r of all buffers with 16-byte peer loads (fp32 accumulate,
//      ranks added in index order, so every rank ends up with bit-identical values) and
//      writes the sums into chunk range r of EVERY rank's buffer with 16-byte peer stores;
//   3. flag barrier B: the last CTA of each rank announces "my writes are done" and waits
//      for the same announcement from every peer before the kernel ends.
// Flags are monotonically increasing epochs (one per call), never reset.  Every spin is
// bounded: on expiry the kernel records a status code and returns, nothing waits for ever.
// Plain loads and stores only — no TMA, no multicast.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.h"
#include "peer_sync.cuh"

namespace b200q {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kThreads = 512;
// 32-bit slots of a rank's flag pad
constexpr int kSlotEpoch = 0;     // number of completed calls
constexpr int kSlotCounter = 1;   // CTAs of this rank that finished the reduce phase
constexpr int kSlotA = 16;        // [kSlotA + src]: src's input is ready (epoch)
constexpr int kSlotB = 32;        // [kSlotB + src]: src's writes are done (epoch)

struct Params {
  void* buf[kMaxWorld];
  unsigned int* pad[kMaxWorld];
  int rank, world;
  unsigned long long n_chunks;  // 16-byte chunks in the tensor
  int is_bf16;
  int* status;
  long long wait_limit;  // SM cycles one wait on a peer may take
};

// W = compile-time bound on the number of ranks, U = chunks per thread per iteration: all
// U * world loads of an iteration are issued before the first use, so that enough bytes are
// in flight to cover the NVLink round trip (small worlds need the larger U).
template <bool BF16, int W, int U>
__global__ void __launch_bounds__(kThreads)
tp_allreduce_kernel(const Params p) {
  __shared__ unsigned int s_epoch;
  __shared__ int s_flag;  // 0 ok, 1 = a wait gave up, 2 = this CTA is the rank's last
  unsigned int* my_pad = p.pad[p.rank];
  if (threadIdx.x == 0) {
    s_epoch = *reinterpret_cast<volatile unsigned int*>(my_pad + kSlotEpoch) + 1u;
    s_flag = 0;
  }
  __syncthreads();
  const unsigned int epoch = s_epoch;

  // ---- barrier A: every rank's partial result is complete
  if (threadIdx.x < p.world) {
    if (blockIdx.x == 0) st_release_sys(p.pad[threadIdx.x] + kSlotA + p.rank, epoch);
    if (!wait_flag(my_pad + kSlotA + threadIdx.x, epoch, p.wait_limit)) s_flag = 1;
  }
  __syncthreads();
  const bool ok = s_flag == 0;

  // ---- reduce my chunk range, publish it to every rank
  if (ok) {
    const unsigned long long per_rank = (p.n_chunks + p.world - 1) / p.world;
    const unsigned long long begin = per_rank * p.rank;
    const unsigned long long end = min(p.n_chunks, begin + per_rank);
    const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * kThreads;
    for (unsigned long long i0 = begin + static_cast<unsigned long long>(blockIdx.x) * kThreads +
                                 threadIdx.x;
         i0 < end; i0 += stride * U) {
      uint4 v[U][W];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const unsigned long long i = i0 + stride * u;
#pragma unroll
        for (int r = 0; r < W; ++r)
          if (r < p.world && i < end) v[u][r] = ld_peer16(static_cast<const uint4*>(p.buf[r]) + i);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const unsigned long long i = i0 + stride * u;
        if (i >= end) break;
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
        for (int r = 0; r < W; ++r)
          if (r < p.world) accumulate<BF16>(acc, v[u][r]);
        const uint4 out = pack<BF16>(acc);
#pragma unroll
        for (int r = 0; r < W; ++r)
          if (r < p.world) st_peer16(static_cast<uint4*>(p.buf[r]) + i, out);
      }
    }
  }
  __threadfence_system();
  __syncthreads();

  // ---- barrier B: by the last CTA of this rank to get here
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(my_pad + kSlotCounter, 1u);
    if (done == gridDim.x - 1) {
      my_pad[kSlotCounter] = 0u;
      s_flag = s_flag == 0 ? 2 : 3;  // 3: this CTA's own wait gave up
    }
  }
  __syncthreads();
  if (s_flag == 2) {
    __threadfence_system();
    if (threadIdx.x < p.world) {
      st_release_sys(p.pad[threadIdx.x] + kSlotB + p.rank, epoch);
      if (!wait_flag(my_pad + kSlotB + threadIdx.x, epoch, p.wait_limit)) atomicCAS(p.status, 0, 0x502);
    }
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned int*>(my_pad + kSlotEpoch) = epoch;
  } else if (s_flag != 0 && threadIdx.x == 0) {
    atomicCAS(p.status, 0, 0x501);
    // Keep the call count in step with the peers even though this call failed.  Only the
    // rank's LAST CTA may do it: every CTA reads the count at its start to learn the call
    // number, so it must not change while a CTA of this launch may still be starting.
    if (s_flag == 3) *reinterpret_cast<volatile unsigned int*>(my_pad + kSlotEpoch) = epoch;
  }
}

// ---------------------------------------------------------------- in-switch reduction
// Same two barriers as the two-shot kernel, but the data phase runs through the NVSwitch's
// multicast/reduction engine (NVLS): one multimem.ld_reduce on the multicast address returns
// the sum of all ranks' values for 16 bytes (fp32 accumulation inside the switch), one
// multimem.st writes the result into every rank's buffer.  Rank r handles slice r.  A GPU
// sends each of its bytes once and receives the full result once, instead of sending and
// receiving (world - 1) / world of the tensor twice: less link traffic from four ranks up.
// All ranks end up with identical bits (one reduction per element, broadcast), but the
// order of the fp32 additions is the switch's, so a result can differ from the rank-ordered
// sum of the other kernels in the last bit.  Plain multimem loads/stores on a multicast
// mapping; no TMA.
template <bool BF16>
__device__ __forceinline__ uint4 multimem_ld_reduce16(const void* mc) {
  uint4 v;
  if (BF16) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
  } else {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
  }
  return v;
}
__device__ __forceinline__ void multimem_st16(void* mc, const uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

template <bool BF16, int U>
__global__ void __launch_bounds__(kThreads)
tp_allreduce_multimem_kernel(const Params p, uint4* __restrict__ mc) {
  __shared__ unsigned int s_epoch;
  __shared__ int s_flag;  // 0 ok, 1 = a wait gave up, 2 = this CTA is the rank's last
  unsigned int* my_pad = p.pad[p.rank];
  if (threadIdx.x == 0) {
    s_epoch = *reinterpret_cast<volatile unsigned int*>(my_pad + kSlotEpoch) + 1u;
    s_flag = 0;
  }
  __syncthreads();
  const unsigned int epoch = s_epoch;
  if (threadIdx.x < p.world) {
    if (blockIdx.x == 0) st_release_sys(p.pad[threadIdx.x] + kSlotA + p.rank, epoch);
    if (!wait_flag(my_pad + kSlotA + threadIdx.x, epoch, p.wait_limit)) s_flag = 1;
  }
  __syncthreads();
  if (s_flag == 0) {
    const unsigned long long per_rank = (p.n_chunks + p.world - 1) / p.world;
    const unsigned long long begin = per_rank * p.rank;
    const unsigned long long end = min(p.n_chunks, begin + per_rank);
    const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * kThreads;
    for (unsigned long long i0 = begin + static_cast<unsigned long long>(blockIdx.x) * kThreads +
                                 threadIdx.x;
         i0 < end; i0 += stride * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const unsigned long long i = i0 + stride * u;
        if (i < end) v[u] = multimem_ld_reduce16<BF16>(mc + i);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const unsigned long long i = i0 + stride * u;
        if (i < end) multimem_st16(mc + i, v[u]);
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(my_pad + kSlotCounter, 1u);
    if (done == gridDim.x - 1) {
      my_pad[kSlotCounter] = 0u;
      s_flag = s_flag == 0 ? 2 : 3;  // 3: this CTA's own wait gave up
    }
  }
  __syncthreads();
  if (s_flag == 2) {
    __threadfence_system();
    if (threadIdx.x < p.world) {
      st_release_sys(p.pad[threadIdx.x] + kSlotB + p.rank, epoch);
      if (!wait_flag(my_pad + kSlotB + threadIdx.x, epoch, p.wait_limit)) atomicCAS(p.status, 0, 0x505);
    }
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned int*>(my_pad + kSlotEpoch) = epoch;
  } else if (s_flag != 0 && threadIdx.x == 0) {
    atomicCAS(p.status, 0, 0x504);
    // only the rank's last CTA moves the call count (see tp_allreduce_kernel)
    if (s_flag == 3) *reinterpret_cast<volatile unsigned int*>(my_pad + kSlotEpoch) = epoch;
  }
}

// ---------------------------------------------------------------- pull variant
// Every rank reads ALL peers' buffers and keeps the sum in a local output tensor: nothing is
// written to a peer, so there is no fence, no acknowledgement to wait for and no closing
// barrier.  Each rank receives (world - 1) x the tensor over NVLink, which equals the two-shot
// scheme's traffic for two ranks (where this variant is used) and exceeds it beyond.
// The inputs must stay untouched until every peer has read them; that is guaranteed by the
// NEXT collective on the same flag pad: a rank announces itself there only after its own
// pull kernel has finished, and nobody passes that announcement barrier without it.  The
// caller therefore alternates between (at least) two input buffers and runs a kernel of
// this file between two writes to the same buffer — which a sequence of row-parallel layers
// does by construction.
template <bool BF16, int W, int U>
__global__ void __launch_bounds__(kThreads)
tp_allreduce_pull_kernel(const Params p, uint4* __restrict__ out) {
  __shared__ unsigned int s_epoch;
  __shared__ int s_flag;
  unsigned int* my_pad = p.pad[p.rank];
  if (threadIdx.x == 0) {
    s_epoch = *reinterpret_cast<volatile unsigned int*>(my_pad + kSlotEpoch) + 1u;
    s_flag = 0;
  }
  __syncthreads();
  const unsigned int epoch = s_epoch;
  if (threadIdx.x < p.world) {
    if (blockIdx.x == 0) st_release_sys(p.pad[threadIdx.x] + kSlotA + p.rank, epoch);
    if (!wait_flag(my_pad + kSlotA + threadIdx.x, epoch, p.wait_limit)) s_flag = 1;
  }
  __syncthreads();
  if (s_flag == 0) {
    const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * kThreads;
    for (unsigned long long i0 = static_cast<unsigned long long>(blockIdx.x) * kThreads + threadIdx.x;
         i0 < p.n_chunks; i0 += stride * U) {
      uint4 v[U][W];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const unsigned long long i = i0 + stride * u;
#pragma unroll
        for (int r = 0; r < W; ++r)
          if (r < p.world && i < p.n_chunks) v[u][r] = ld_peer16(static_cast<const uint4*>(p.buf[r]) + i);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const unsigned long long i = i0 + stride * u;
        if (i >= p.n_chunks) break;
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
        for (int r = 0; r < W; ++r)
          if (r < p.world) accumulate<BF16>(acc, v[u][r]);
        out[i] = pack<BF16>(acc);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_flag != 0) atomicCAS(p.status, 0, 0x503);
    // the rank's last CTA publishes the finished call number (the next launch reads it)
    if (atomicAdd(my_pad + kSlotCounter, 1u) == gridDim.x - 1) {
      my_pad[kSlotCounter] = 0u;
      *reinterpret_cast<volatile unsigned int*>(my_pad + kSlotEpoch) = epoch;
    }
  }
}

// ---------------------------------------------------------------- small tensors, one trip
// For tensors of up to a few hundred kilobytes the two barriers above cost more than the
// data.  Here every rank pushes its whole tensor to every peer as tagged 8-byte words and
// then sums what it received, in rank order: one NVLink trip, no fence, no flag.  Shares
// the receive area, the parity halves and the call numbering with the fused decode kernels
// (the same argument shows that no rank overwrites words a peer still reads).  x and y are
// ordinary local tensors (y may be x).  CTA c of every rank handles the same chunk range,
// and all CTAs are resident, so no CTA waits for one that cannot run.
struct OneTripParams {
  void* recv[kMaxWorld];
  unsigned int* ctl;   // this rank's control words
  size_t half_bytes;
  const uint4* x;
  uint4* y;
  unsigned long long n_chunks;
  int rank, world;
  int* status;
  long long wait_limit;
};

template <bool BF16>
__global__ void __launch_bounds__(kThreads)
tp_allreduce_onetrip_kernel(const OneTripParams p) {
  __shared__ unsigned int s_epoch;
  __shared__ int s_fail;
  if (threadIdx.x == 0) {
    s_epoch = next_epoch(p.ctl);
    s_fail = 0;
  }
  __syncthreads();
  const unsigned int epoch = s_epoch;
  const size_t half_off = (epoch & 1u) * p.half_bytes;
  const unsigned long long slot_words = p.n_chunks * 4;
  const unsigned long long first = static_cast<unsigned long long>(blockIdx.x) * kThreads + threadIdx.x;
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * kThreads;

  for (unsigned long long c = first; c < p.n_chunks; c += stride) {
    const uint4 v = p.x[c];
    for (int peer = 0; peer < p.world; ++peer) {
      if (peer == p.rank) continue;
      uint2* dst = reinterpret_cast<uint2*>(static_cast<char*>(p.recv[peer]) + half_off) +
                   p.rank * slot_words + c * 4;
      st_word8(dst + 0, v.x, epoch);
      st_word8(dst + 1, v.y, epoch);
      st_word8(dst + 2, v.z, epoch);
      st_word8(dst + 3, v.w, epoch);
    }
  }
  const uint2* mine = reinterpret_cast<const uint2*>(static_cast<const char*>(p.recv[p.rank]) + half_off);
  bool ok = true;
  for (unsigned long long c = first; c < p.n_chunks; c += stride) {
    const uint4 own = p.x[c];
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int r = 0; r < p.world; ++r) {
      uint4 v = own;
      if (r != p.rank) {
        const uint2* src = mine + r * slot_words + c * 4;
        ok &= wait_word8(src + 0, epoch, &v.x, p.wait_limit);
        ok &= wait_word8(src + 1, epoch, &v.y, p.wait_limit);
        ok &= wait_word8(src + 2, epoch, &v.z, p.wait_limit);
        ok &= wait_word8(src + 3, epoch, &v.w, p.wait_limit);
      }
      accumulate<BF16>(acc, v);
    }
    if (ok) p.y[c] = pack<BF16>(acc);
  }
  if (!ok) s_fail = 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_fail != 0) atomicCAS(p.status, 0, 0x602);
    finish_call(p.ctl, epoch);
  }
}

// ------------------------------------------------- second half of the fused prefill all-reduce
// The scatter GEMMs (gemm_umma_pair.cu) have put every rank's partial tiles for the token
// rows this rank owns into the local staging area.  This kernel first exchanges one flag per
// peer ("my scatter GEMM has completed": true by stream order when this kernel starts),
// then sums the `world` partials in rank order in fp32 — local loads only — and writes the
// result rows into EVERY rank's output matrix with 16-byte peer stores (the all-gather
// half).  It ends with the same "my writes are done" barrier as the two-shot kernel, using
// the shared call numbering of the tagged-word kernels.
constexpr int kCtlReady = 24;  // control words [kCtlReady + src]: src's scatter GEMM is complete
constexpr int kCtlDone = 16;  // control words [kCtlDone + src]: src finished writing (call number)

struct GatherParams {
  const void* stage;           // local staging: [src][rows_per_owner][N] values
  void* y[kMaxWorld];          // every rank's output matrix [M][N]
  unsigned int* ctl[kMaxWorld];
  int rank, world;
  int rows_per_owner, N, tiles_b;
  int* status;
  long long wait_limit;
};

// W = compile-time bound on the number of ranks, U = chunks per thread in flight (U * W loads
// are issued before the first use).
template <bool BF16, int W, int U>
__global__ void __launch_bounds__(kThreads)
tp_reduce_gather_kernel(const GatherParams p) {
  __shared__ unsigned int s_epoch;
  __shared__ int s_flag;  // 0 ok, 1 = a wait gave up, 2 / 3 = this CTA is the rank's last (ok / failed)
  unsigned int* ctl = p.ctl[p.rank];
  if (threadIdx.x == 0) {
    s_epoch = next_epoch(ctl);
    s_flag = 0;
  }
  __syncthreads();
  const unsigned int epoch = s_epoch;
  const int row_blocks = p.rows_per_owner / 128;
  const int n_tiles = row_blocks * p.tiles_b;
  const size_t slot_chunks = static_cast<size_t>(p.rows_per_owner) * p.N / 8;
  const int row_chunks = p.N / 8;  // 16-byte chunks per matrix row
  const uint4* stage = static_cast<const uint4*>(p.stage);

  // every rank's scatter GEMM has completed (stream order on the sender, one flag per peer)
  if (threadIdx.x < p.world) {
    if (blockIdx.x == 0) st_release_sys(p.ctl[threadIdx.x] + kCtlReady + p.rank, epoch);
    if (!wait_flag(ctl + kCtlReady + threadIdx.x, epoch, p.wait_limit)) s_flag = 1;
  }
  __syncthreads();
  const bool ready = s_flag == 0;
  for (int t = blockIdx.x; ready && t < n_tiles; t += gridDim.x) {
    const int block = t / p.tiles_b, tile_b = t - block * p.tiles_b;
    // 128 rows x 32 chunks of 16 bytes, U chunks per thread per round
    for (int c0 = threadIdx.x; c0 < 128 * 32; c0 += kThreads * U) {
      uint4 v[U][W];
      size_t off[U];
      bool live[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = c0 + u * kThreads;
        const int r = c >> 5, cc = (c & 31) + tile_b * 32;
        live[u] = c < 128 * 32 && cc < row_chunks;
        off[u] = static_cast<size_t>(block * 128 + r) * row_chunks + cc;
#pragma unroll
        for (int src = 0; src < W; ++src)
          if (src < p.world && live[u]) v[u][src] = ld_volatile16(stage + src * slot_chunks + off[u]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (!live[u]) continue;
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
        for (int src = 0; src < W; ++src)
          if (src < p.world) accumulate<BF16>(acc, v[u][src]);
        const uint4 out = pack<BF16>(acc);
        const size_t yoff = static_cast<size_t>(p.rank) * slot_chunks + off[u];
#pragma unroll
        for (int dst = 0; dst < W; ++dst)
          if (dst < p.world) st_peer16(static_cast<uint4*>(p.y[dst]) + yoff, out);
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(ctl + kCtlCounter, 1u);
    if (done == gridDim.x - 1) {
      ctl[kCtlCounter] = 0u;
      s_flag = s_flag == 0 ? 2 : 3;
    }
  }
  __syncthreads();
  if (s_flag >= 2) {
    __threadfence_system();
    if (threadIdx.x < p.world) {
      st_release_sys(p.ctl[threadIdx.x] + kCtlDone + p.rank, epoch);
      if (!wait_flag(ctl + kCtlDone + threadIdx.x, epoch, p.wait_limit)) atomicCAS(p.status, 0, 0x702);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      if (s_flag == 3) atomicCAS(p.status, 0, 0x701);
      *reinterpret_cast<volatile unsigned int*>(ctl + kCtlEpoch) = epoch;
    }
  } else if (s_flag == 1 && threadIdx.x == 0) {
    atomicCAS(p.status, 0, 0x701);
  }
}

}  // namespace

int launch_tp_reduce_gather(const void* stage, void* const* peer_y,
                            void* const* peer_ctl, int rank, int world, int M, int N, int dtype,
                            cudaStream_t stream) {
  GatherParams p{};
  p.stage = stage;
  for (int r = 0; r < world; ++r) {
    p.y[r] = peer_y[r];
    p.ctl[r] = static_cast<unsigned int*>(peer_ctl[r]);
  }
  p.rank = rank;
  p.world = world;
  p.rows_per_owner = M / world;
  p.N = N;
  p.tiles_b = (N + 255) / 256;
  p.status = device_status_ptr();
  p.wait_limit = peer_wait_limit_cycles();
  if (p.status == nullptr) return B200Q_ERR_LAUNCH;
  const int n_tiles = (p.rows_per_owner / 128) * p.tiles_b;
  const int grid = n_tiles < sm_count() ? n_tiles : sm_count();
#define B200Q_RG_LAUNCH(BF, W, U) tp_reduce_gather_kernel<BF, W, U><<<grid, kThreads, 0, stream>>>(p)
  if (dtype == B200Q_DTYPE_BF16) {
    if (world <= 2) B200Q_RG_LAUNCH(true, 2, 8);
    else if (world <= 4) B200Q_RG_LAUNCH(true, 4, 4);
    else B200Q_RG_LAUNCH(true, 8, 2);
  } else {
    if (world <= 2) B200Q_RG_LAUNCH(false, 2, 8);
    else if (world <= 4) B200Q_RG_LAUNCH(false, 4, 4);
    else B200Q_RG_LAUNCH(false, 8, 2);
  }
#undef B200Q_RG_LAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch();
  return B200Q_OK;
}

}  // namespace b200q

extern "C" int b200q_tp_allreduce(void* const* peer_buffers, void* const* peer_flag_pads, int rank,
                                  int world, size_t n_elems, int dtype, void* stream) {
  using namespace b200q;
  if (peer_buffers == nullptr || peer_flag_pads == nullptr) return B200Q_ERR_NULL_POINTER;
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return B200Q_ERR_BAD_ARGUMENT;
  if (dtype != B200Q_DTYPE_F16 && dtype != B200Q_DTYPE_BF16) return B200Q_ERR_BAD_ARGUMENT;
  if (n_elems == 0 || (n_elems % 8) != 0) return B200Q_ERR_UNSUPPORTED_SHAPE;  // 16-byte chunks
  Params p{};
  for (int r = 0; r < world; ++r) {
    if (peer_buffers[r] == nullptr || peer_flag_pads[r] == nullptr) return B200Q_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(peer_buffers[r]) & 15u) != 0) return B200Q_ERR_MISALIGNED;
    p.buf[r] = peer_buffers[r];
    p.pad[r] = static_cast<unsigned int*>(peer_flag_pads[r]);
  }
  if (device_cc_major() != 10) return B200Q_ERR_UNSUPPORTED_ARCH;
  p.rank = rank;
  p.world = world;
  p.n_chunks = n_elems / 8;
  p.is_bf16 = dtype == B200Q_DTYPE_BF16;
  p.status = device_status_ptr();
  p.wait_limit = peer_wait_limit_cycles();
  if (p.status == nullptr) return B200Q_ERR_LAUNCH;
  const unsigned long long per_rank = (p.n_chunks + world - 1) / world;
  long long blocks = static_cast<long long>((per_rank + kThreads * 4 - 1) / (kThreads * 4));
  if (blocks < 1) blocks = 1;
  if (blocks > sm_count()) blocks = sm_count();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = static_cast<int>(blocks);
#define B200Q_AR_LAUNCH(BF, W, U) tp_allreduce_kernel<BF, W, U><<<grid, kThreads, 0, st>>>(p)
  if (p.is_bf16) {
    if (world <= 2) B200Q_AR_LAUNCH(true, 2, 4);
    else if (world <= 4) B200Q_AR_LAUNCH(true, 4, 2);
    else B200Q_AR_LAUNCH(true, 8, 1);
  } else {
    if (world <= 2) B200Q_AR_LAUNCH(false, 2, 4);
    else if (world <= 4) B200Q_AR_LAUNCH(false, 4, 2);
    else B200Q_AR_LAUNCH(false, 8, 1);
  }
#undef B200Q_AR_LAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch();
  return B200Q_OK;
}

extern "C" int b200q_tp_allreduce_small(const void* x, void* y, size_t n_elems, int dtype,
                                        void* const* peer_recv, void* const* peer_flags,
                                        size_t recv_bytes, int rank, int world, void* stream) {
  using namespace b200q;
  if (x == nullptr || y == nullptr || peer_recv == nullptr || peer_flags == nullptr)
    return B200Q_ERR_NULL_POINTER;
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return B200Q_ERR_BAD_ARGUMENT;
  if (dtype != B200Q_DTYPE_F16 && dtype != B200Q_DTYPE_BF16) return B200Q_ERR_BAD_ARGUMENT;
  if (n_elems == 0 || (n_elems % 8) != 0) return B200Q_ERR_UNSUPPORTED_SHAPE;
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) != 0)
    return B200Q_ERR_MISALIGNED;
  OneTripParams p{};
  const size_t half = (recv_bytes / 2) & ~static_cast<size_t>(255);
  if (static_cast<size_t>(world) * n_elems * 4 > half) return B200Q_ERR_WORKSPACE;
  for (int r = 0; r < world; ++r) {
    if (peer_recv[r] == nullptr || peer_flags[r] == nullptr) return B200Q_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(peer_recv[r]) & 255u) != 0) return B200Q_ERR_MISALIGNED;
    p.recv[r] = peer_recv[r];
  }
  if (device_cc_major() != 10) return B200Q_ERR_UNSUPPORTED_ARCH;
  p.ctl = static_cast<unsigned int*>(peer_flags[rank]);
  p.half_bytes = half;
  p.x = static_cast<const uint4*>(x);
  p.y = static_cast<uint4*>(y);
  p.n_chunks = n_elems / 8;
  p.rank = rank;
  p.world = world;
  p.status = device_status_ptr();
  p.wait_limit = peer_wait_limit_cycles();
  if (p.status == nullptr) return B200Q_ERR_LAUNCH;
  // one chunk per thread until every SM has a CTA; never more CTAs than are resident at once
  long long blocks = static_cast<long long>((p.n_chunks + kThreads - 1) / kThreads);
  if (blocks > sm_count()) blocks = sm_count();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B200Q_DTYPE_BF16) {
    tp_allreduce_onetrip_kernel<true><<<static_cast<int>(blocks), kThreads, 0, st>>>(p);
  } else {
    tp_allreduce_onetrip_kernel<false><<<static_cast<int>(blocks), kThreads, 0, st>>>(p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch();
  return B200Q_OK;
}

extern "C" int b200q_tp_allreduce_pull(void* const* peer_buffers, void* const* peer_flag_pads,
                                       void* out, int rank, int world, size_t n_elems, int dtype,
                                       void* stream) {
  using namespace b200q;
  if (peer_buffers == nullptr || peer_flag_pads == nullptr || out == nullptr)
    return B200Q_ERR_NULL_POINTER;
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return B200Q_ERR_BAD_ARGUMENT;
  if (dtype != B200Q_DTYPE_F16 && dtype != B200Q_DTYPE_BF16) return B200Q_ERR_BAD_ARGUMENT;
  if (n_elems == 0 || (n_elems % 8) != 0) return B200Q_ERR_UNSUPPORTED_SHAPE;
  if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0) return B200Q_ERR_MISALIGNED;
  Params p{};
  for (int r = 0; r < world; ++r) {
    if (peer_buffers[r] == nullptr || peer_flag_pads[r] == nullptr) return B200Q_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(peer_buffers[r]) & 15u) != 0) return B200Q_ERR_MISALIGNED;
    p.buf[r] = peer_buffers[r];
    p.pad[r] = static_cast<unsigned int*>(peer_flag_pads[r]);
  }
  if (out == peer_buffers[rank]) return B200Q_ERR_BAD_ARGUMENT;  // peers still read the input
  if (device_cc_major() != 10) return B200Q_ERR_UNSUPPORTED_ARCH;
  p.rank = rank;
  p.world = world;
  p.n_chunks = n_elems / 8;
  p.is_bf16 = dtype == B200Q_DTYPE_BF16;
  p.status = device_status_ptr();
  p.wait_limit = peer_wait_limit_cycles();
  if (p.status == nullptr) return B200Q_ERR_LAUNCH;
  long long blocks = static_cast<long long>((p.n_chunks + kThreads * 4 - 1) / (kThreads * 4));
  if (blocks < 1) blocks = 1;
  if (blocks > 2 * sm_count()) blocks = 2 * sm_count();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = static_cast<int>(blocks);
  uint4* o = static_cast<uint4*>(out);
#define B200Q_PULL_LAUNCH(BF, W, U) tp_allreduce_pull_kernel<BF, W, U><<<grid, kThreads, 0, st>>>(p, o)
  if (p.is_bf16) {
    if (world <= 2) B200Q_PULL_LAUNCH(true, 2, 8);
    else if (world <= 4) B200Q_PULL_LAUNCH(true, 4, 2);
    else B200Q_PULL_LAUNCH(true, 8, 1);
  } else {
    if (world <= 2) B200Q_PULL_LAUNCH(false, 2, 8);
    else if (world <= 4) B200Q_PULL_LAUNCH(false, 4, 2);
    else B200Q_PULL_LAUNCH(false, 8, 1);
  }
#undef B200Q_PULL_LAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch();
  return B200Q_OK;
}

extern "C" int b200q_tp_allreduce_multimem(void* multicast_buffer, void* const* peer_flag_pads,
                                           int rank, int world, size_t n_elems, int dtype,
                                           void* stream) {
  using namespace b200q;
  if (multicast_buffer == nullptr || peer_flag_pads == nullptr) return B200Q_ERR_NULL_POINTER;
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return B200Q_ERR_BAD_ARGUMENT;
  if (dtype != B200Q_DTYPE_F16 && dtype != B200Q_DTYPE_BF16) return B200Q_ERR_BAD_ARGUMENT;
  if (n_elems == 0 || (n_elems % 8) != 0) return B200Q_ERR_UNSUPPORTED_SHAPE;
  if ((reinterpret_cast<uintptr_t>(multicast_buffer) & 15u) != 0) return B200Q_ERR_MISALIGNED;
  Params p{};
  for (int r = 0; r < world; ++r) {
    if (peer_flag_pads[r] == nullptr) return B200Q_ERR_NULL_POINTER;
    p.pad[r] = static_cast<unsigned int*>(peer_flag_pads[r]);
  }
  if (device_cc_major() != 10) return B200Q_ERR_UNSUPPORTED_ARCH;
  p.rank = rank;
  p.world = world;
  p.n_chunks = n_elems / 8;
  p.is_bf16 = dtype == B200Q_DTYPE_BF16;
  p.status = device_status_ptr();
  p.wait_limit = peer_wait_limit_cycles();
  if (p.status == nullptr) return B200Q_ERR_LAUNCH;
  const unsigned long long per_rank = (p.n_chunks + world - 1) / world;
  long long blocks = static_cast<long long>((per_rank + kThreads * 4 - 1) / (kThreads * 4));
  if (blocks < 1) blocks = 1;
  if (blocks > sm_count()) blocks = sm_count();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint4* mc = static_cast<uint4*>(multicast_buffer);
  if (p.is_bf16) {
    tp_allreduce_multimem_kernel<true, 4><<<static_cast<int>(blocks), kThreads, 0, st>>>(p, mc);
  } else {
    tp_allreduce_multimem_kernel<false, 4><<<static_cast<int>(blocks), kThreads, 0, st>>>(p, mc);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch();
  return B200Q_OK;
}
