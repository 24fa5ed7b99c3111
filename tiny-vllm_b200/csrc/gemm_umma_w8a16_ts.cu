// W8A16 prefill GEMM with the weights as the tensor-memory A operand of tcgen05.mma.
//
// The shared-memory kernel (gemm_umma_w8a16.cu) is bound by shared-memory traffic: per
// 64-element K block of a 128 x 256 tile it moves 128 KB (TMA writes, the expansion's read
// and 16-bit write, the tensor core's read of both operands).  Here the expanded weights
// never touch shared memory: the converter warps write them straight into tensor memory
// (tcgen05.st) and the MMA takes its A operand from there, so a block costs 80 KB for the
// same number of flops.
//
// Tile of one CTA: 256 output channels (two A tiles of 128 rows) x 128 tokens (B, shared by
// both MMAs).  Tensor memory (512 columns): accumulators 2 x 128 columns (channel tile 0 / 1,
// lane = channel, column = token), A ring 4 stages x 2 tiles x 32 columns.  All columns are
// in use, so the accumulators are single-buffered: the epilogue of a tile does not overlap
// the main loop of the next.
//
// Warp roles (832 threads, 1 CTA per SM, persistent):
//   warp 0      TMA producer: token tile (128 x 128 B, 128-byte swizzle) + raw int8 tile
//               (256 x 64 B, 64-byte swizzle) per K block of 64 elements
//   warp 1      UMMA issuer (one thread): 2 x 4 tcgen05.mma (A from tensor memory) per block
//   warps 2-9   epilogue, four warps per channel tile: tcgen05.ld -> acc * s[n] + b[n] ->
//               16 bit -> y[token][channel]
//   warps 10-25 converters, two groups of eight taking K blocks in turn: warp w owns TMEM
//               lanes 32 (w % 4) .. + 31 of one channel tile: one raw row per thread -> 32
//               packed words -> tcgen05.st
// Every mbarrier wait is bounded.  Arithmetic as in the shared-memory kernel: fp32 sums of
// x * float(q), then acc * s[n] + b[n]
// (nanovllm/quantization/csrc/int8_weight_only_gemm.cu:258-292, 397-412).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "common.h"
#include "ptx_sm100.cuh"
#include "w8a16_device.cuh"

namespace b200q {
namespace {

constexpr int kTsChannels = 256;   // output channels per CTA tile (two A tiles)
constexpr int kTsTokens = 128;     // tokens per CTA tile (UMMA N)
constexpr int kTsTokBytes = kTsTokens * kRow16;     // 16 KB
constexpr int kTsRawBytes = kTsChannels * kRow8;    // 16 KB
constexpr int kTsStageBytes = kTsTokBytes + kTsRawBytes;
constexpr int kTsStages = 6;
constexpr int kTsAStages = 4;
constexpr int kTsCtrlBytes = 512;
// epilogue staging: per channel tile two buffers of 32 tokens x 128 channels, 16 bit
constexpr int kTsStageOutBytes = 32 * kTileA * 2;
constexpr int kTsEpiWarps = 8;     // four per channel tile (one per TMEM lane quarter)
constexpr int kTsEpiThreads = kTsEpiWarps * 32;
constexpr int kTsSmem = kTsStages * kTsStageBytes + 4 * kTsStageOutBytes + kTsCtrlBytes;
constexpr int kTsTmemCols = 512;
constexpr int kTsConvGroups = 2;   // converter groups taking K blocks in turn
constexpr int kTsThreads = 64 + kTsEpiThreads + kTsConvGroups * kConvThreads;  // 832
constexpr int kTsAcol0 = 256;      // first column of the A ring
constexpr int kTsAStageCols = 64;  // two tiles x 32 columns

struct TsParams {
  int M, N, K;                 // tokens, channels, features
  int tiles_ch, tiles_tok, k_blocks;
  int is_bf16;
  const float* w_scales;
  const void* bias;
  void* out;
  int* status;
  int debug_flags;             // test-only: 1 = skip epilogue work, 8 = skip the expansion
};

template <typename T>
__global__ void __launch_bounds__(kTsThreads, 1)
w8a16_umma_ts_kernel(const __grid_constant__ CUtensorMap tmap_x,
                     const __grid_constant__ CUtensorMap tmap_w, const TsParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* out_stage = smem + kTsStages * kTsStageBytes;
  uint8_t* ctrl = out_stage + 4 * kTsStageOutBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);   // [stages] TMA bytes landed
  uint64_t* empty_bar = full_bar + kTsStages;               // [stages] MMAs that read it are done
  uint64_t* afull_bar = empty_bar + kTsStages;              // [a stages] expansion written
  uint64_t* aempty_bar = afull_bar + kTsAStages;            // [a stages] MMAs that read it are done
  uint64_t* tfull_bar = aempty_bar + kTsAStages;            // accumulators complete
  uint64_t* tempty_bar = tfull_bar + 1;                     // accumulators drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = ptx::smem_u32(smem);
  if ((smem_base & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, 0x200);
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTsStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(full_bar + s), 1);
      ptx::mbar_init(ptx::smem_u32(empty_bar + s), 1);
    }
    for (int s = 0; s < kTsAStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(afull_bar + s), kConvWarps);
      ptx::mbar_init(ptx::smem_u32(aempty_bar + s), 1);
    }
    ptx::mbar_init(ptx::smem_u32(tfull_bar), 1);
    ptx::mbar_init(ptx::smem_u32(tempty_bar), kTsEpiThreads);
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::tma_prefetch_desc(&tmap_x);
    ptx::tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTsTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // everything above overlapped the previous kernel's tail; its results are needed from here
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();

  const int total_items = p.tiles_ch * p.tiles_tok;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------ TMA producer
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const int tile_ch = item % p.tiles_ch;    // channel tiles fastest: neighbours share tokens
        const int tile_tok = item / p.tiles_ch;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(empty_bar + stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t bar = ptx::smem_u32(full_bar + stage);
          const uint32_t s16 = smem_base + stage * kTsStageBytes;
          ptx::mbar_arrive_expect_tx(bar, kTsStageBytes);
          ptx::tma_load_2d(s16, &tmap_x, bar, kb * kBlockK * 2, tile_tok * kTsTokens);
          ptx::tma_load_2d(s16 + kTsTokBytes, &tmap_w, bar, kb * kBlockK, tile_ch * kTsChannels);
          if (++stage == kTsStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------- UMMA issuer
      const uint32_t idesc = ptx::umma_idesc(1u, p.is_bf16 ? 1u : 0u, kTileA, kTsTokens);
      int stage = 0, as = 0;
      uint32_t phase = 0, aphase = 0;
      int it = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x, ++it) {
        // single accumulator set: wait until the epilogue of the previous tile has drained it
        if (!ptx::mbar_wait(ptx::smem_u32(tempty_bar), (static_cast<uint32_t>(it) & 1u) ^ 1u, abort_flag))
          break;
        ptx::tc_fence_after_sync();
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(full_bar + stage), phase, abort_flag) ||
              !ptx::mbar_wait(ptx::smem_u32(afull_bar + as), aphase, abort_flag)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint64_t b_desc = ptx::umma_desc_k_sw128(smem_base + stage * kTsStageBytes);
          const uint32_t a0 = tmem_base + kTsAcol0 + as * kTsAStageCols;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
            ptx::umma_f16_ts(tmem_base, a0 + 8u * k, b_desc + 2u * k, idesc, acc);
            ptx::umma_f16_ts(tmem_base + kTsTokens, a0 + 32u + 8u * k, b_desc + 2u * k, idesc, acc);
          }
          ptx::umma_commit(ptx::smem_u32(empty_bar + stage));
          ptx::umma_commit(ptx::smem_u32(aempty_bar + as));
          if (++stage == kTsStages) {
            stage = 0;
            phase ^= 1u;
          }
          if (++as == kTsAStages) {
            as = 0;
            aphase ^= 1u;
          }
        }
        if (ok) ptx::umma_commit(ptx::smem_u32(tfull_bar));
      }
    }
  } else if (warp >= 2 + kTsEpiWarps) {
    // ---------------------------------------------------------- converters
    // One K block is a dependent chain per thread (wait, 4 loads, expansion, tcgen05.st, wait,
    // arrive); two groups of eight warps take the blocks in turn so that two chains overlap.
    const int cw = warp - (2 + kTsEpiWarps);     // 0..15
    const int group = cw >> 3;                   // blocks group, group + 2, ...
    const int tile = (cw & 7) >> 2;              // channel tile of this warp
    const int quarter = warp & 3;                // TMEM lane quarter this warp may access
    const int r = tile * kTileA + quarter * 32 + lane;  // raw row (channel) of this thread
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kTsAcol0 +
                               static_cast<uint32_t>(tile * 32);
    uint32_t blk = 0;  // K blocks seen so far, over all items
    bool ok = true;
    for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
      for (int kb = 0; kb < p.k_blocks; ++kb, ++blk) {
        if (static_cast<int>(blk & 1u) != group) continue;
        const uint32_t stage = blk % kTsStages, phase = (blk / kTsStages) & 1u;
        const uint32_t as = blk % kTsAStages, aphase = (blk / kTsAStages) & 1u;
        if (!ptx::mbar_wait(ptx::smem_u32(full_bar + stage), phase, abort_flag) ||
            !ptx::mbar_wait(ptx::smem_u32(aempty_bar + as), aphase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint8_t* src_row = smem + stage * kTsStageBytes + kTsTokBytes + r * kRow8;
        const int sw8 = (r >> 1) & 3;
        uint32_t v[32];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 w = make_uint4(0u, 0u, 0u, 0u);
          if (!(p.debug_flags & 8)) w = *reinterpret_cast<const uint4*>(src_row + ((c ^ sw8) << 4));
          const uint2 e0 = expand4<T>(w.x), e1 = expand4<T>(w.y), e2 = expand4<T>(w.z),
                      e3 = expand4<T>(w.w);
          v[8 * c + 0] = e0.x;
          v[8 * c + 1] = e0.y;
          v[8 * c + 2] = e1.x;
          v[8 * c + 3] = e1.y;
          v[8 * c + 4] = e2.x;
          v[8 * c + 5] = e2.y;
          v[8 * c + 6] = e3.x;
          v[8 * c + 7] = e3.y;
        }
        ptx::tmem_st_32x32b_x32(lane_base + as * kTsAStageCols, v);
        ptx::tmem_st_wait();
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(afull_bar + as));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    // A thread holds one channel (its TMEM lane) and 32 tokens per load, but y is token-major:
    // the four warps of a channel tile put their 32 x 32 blocks side by side in shared memory
    // as [token][128 channels] and then write whole 256-byte token rows, 16 bytes per lane.
    // Warps 2-5 drain channel tile 0, warps 6-9 channel tile 1, at the same time.
    const int quarter = warp & 3;
    const int t = (warp - 2) >> 2;                // channel tile of this warp
    const int sub = (warp - 2) & 3;               // warp inside its group of four
    const T* bias = reinterpret_cast<const T*>(p.bias);
    T* out = reinterpret_cast<T*>(p.out);
    uint8_t* my_stage = out_stage + t * 2 * kTsStageOutBytes;
    int it = 0, round = 0;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it) {
      const int tile_ch = item % p.tiles_ch;
      const int tile_tok = item / p.tiles_ch;
      if (!ptx::mbar_wait(ptx::smem_u32(tfull_bar), static_cast<uint32_t>(it) & 1u, abort_flag)) break;
      ptx::tc_fence_after_sync();
      const int ch0 = tile_ch * kTsChannels + t * kTileA;       // first channel of this A tile
      const int ch = ch0 + quarter * 32 + lane;
      const bool ch_ok = ch < p.N;
      const float s = ch_ok ? __ldg(p.w_scales + ch) : 0.f;
      const float b = (ch_ok && bias != nullptr) ? to_float<T>(bias[ch]) : 0.f;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(t * kTsTokens);
#pragma unroll 1
      for (int c = 0; c < kTsTokens / 32; ++c, ++round) {
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(taddr + c * 32, v);
        ptx::tmem_ld_wait();
        if (p.debug_flags & 1) continue;
        T* buf = reinterpret_cast<T*>(my_stage + (round & 1) * kTsStageOutBytes);
#pragma unroll
        for (int j = 0; j < 32; ++j)
          buf[j * kTileA + quarter * 32 + lane] = from_float<T>(scale_acc(__uint_as_float(v[j]), s, b));
        // all four blocks are in place; passing this barrier also means that every warp of the
        // group has finished reading the other buffer (it did so before arriving here)
        ptx::named_bar_sync(2 + t, kEpiThreads);
        const int tok0 = tile_tok * kTsTokens + c * 32;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int j = sub * 8 + i * 2 + (lane >> 4);       // token row inside the chunk
          const int col = (lane & 15) * 8;                   // first of 8 channels
          const int tok = tok0 + j;
          if (tok < p.M && ch0 + col < p.N)                   // N % 8 == 0: all in or all out
            *reinterpret_cast<uint4*>(out + static_cast<size_t>(tok) * p.N + ch0 + col) =
                *reinterpret_cast<const uint4*>(buf + j * kTileA + col);
        }
      }
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(ptx::smem_u32(tempty_bar));
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTsTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag != 0) {
    atomicCAS(p.status, 0, 0x900 | (static_cast<int>(blockIdx.x) << 12));
  }
}

template <typename T>
cudaError_t launch_ts(const CUtensorMap& tx, const CUtensorMap& tw, const TsParams& tp, int grid,
                      cudaStream_t stream) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = w8a16_umma_ts_kernel<T>;
  if (dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kTsSmem);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  return launch_overlapped(kern, grid, kTsThreads, kTsSmem, stream, tx, tw, tp);
}

}  // namespace

// Prefill-sized problems with enough 256 x 128 tiles to fill the GPU and at least 16 K blocks:
// the epilogue of a tile is not overlapped here (all of tensor memory is in use), so very short
// K loops stay on the shared-memory kernel.  M = 8192, this kernel vs that one: 1024 -> 4096
// 84.3 vs 87.1 us, 2048 -> 1024 44.8 vs 49.9 us, 1024 -> 6144 128.4 vs 131.5 us, 3072 -> 1024
// 61.6 vs 71.3 us.
bool umma16_ts_applicable(int M, int N, int K) {
  if (debug_knob(B200Q_KNOB_NO_TS, 0) != 0) return false;
  if (K < debug_knob(B200Q_KNOB_TS_MIN_K, 1024)) return false;
  if ((K % 16) != 0 || (N % 8) != 0) return false;   // 16-byte output pieces
  const long long tiles = static_cast<long long>((N + kTsChannels - 1) / kTsChannels) *
                          ((M + kTsTokens - 1) / kTsTokens);
  return M >= 512 && tiles >= sm_count();
}

int launch_w8a16_umma_ts(const GemmArgs& a) {
  CUtensorMap tx, tw;
  if (!make_tensor_map(a.x, a.M, static_cast<uint64_t>(a.K) * 2, kTsTokens, kRow16, &tx))
    return B200Q_ERR_LAUNCH;
  if (!get_tensor_map(a.w, a.N, a.K, kTsChannels, kRow8, &tw)) return B200Q_ERR_LAUNCH;
  TsParams tp{};
  tp.M = a.M;
  tp.N = a.N;
  tp.K = a.K;
  tp.tiles_ch = (a.N + kTsChannels - 1) / kTsChannels;
  tp.tiles_tok = (a.M + kTsTokens - 1) / kTsTokens;
  tp.k_blocks = (a.K + kBlockK - 1) / kBlockK;
  tp.is_bf16 = a.dtype == B200Q_DTYPE_BF16 ? 1 : 0;
  tp.w_scales = a.w_scales;
  tp.bias = a.bias;
  tp.out = a.y;
  tp.status = a.status;
  tp.debug_flags = debug_knob(B200Q_KNOB_FLAGS, 0);
  const long long items = static_cast<long long>(tp.tiles_ch) * tp.tiles_tok;
  const int grid = static_cast<int>(std::min<long long>(items, sm_count()));
  cudaError_t e = a.dtype == B200Q_DTYPE_BF16 ? launch_ts<__nv_bfloat16>(tx, tw, tp, grid, a.stream)
                                              : launch_ts<__half>(tx, tw, tp, grid, a.stream);
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch();
  return B200Q_OK;
}

}  // namespace b200q
