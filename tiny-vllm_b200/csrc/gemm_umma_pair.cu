// W8A8 prefill GEMM on CTA pairs: tcgen05.mma.cta_group::2, 256 x 256 output tile per pair.
//
// Two CTAs on neighbouring SMs (a cluster of two) share one UMMA: each CTA loads its own
// 128 token rows of A and HALF of the 256 weight rows of B per K block (32 KB instead of
// the 48 KB a single-CTA 128 x 256 tile needs), the leader CTA issues the MMAs for both,
// and each CTA finds its 128 x 256 accumulator in its own TMEM.  That cuts the L2 -> SM
// traffic per output by a third and lets the ring hold six stages instead of four, which
// is what the single-CTA kernel is limited by at these shapes.
//
// No data travels between the two CTAs except through the tensor core's operand fetch:
// every TMA load lands in the issuing CTA's own shared memory; only its completion is
// counted on the leader's mbarrier.  Cross-CTA signals:
//   full[s]    (leader)      <- TMA transaction bytes of both CTAs
//   empty[s]   (each CTA)    <- one tcgen05.commit per CTA, issued by the leader
//   tfull[b]   (each CTA)    <- one tcgen05.commit per CTA, issued by the leader
//   tempty[b]  (leader)      <- epilogue threads of both CTAs (remote mbarrier arrive)
// Every mbarrier wait is bounded; the two cluster-wide hardware barriers (after set-up,
// before tear-down) are reached by every thread on every path.
//
// Arithmetic: exact int32 accumulation, then (float(acc) * a_s[m]) * w_s[n] + bias[n]
// (nanovllm/quantization/csrc/w8a8_gemm.cu:165-183, 387-390).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "common.h"
#include "ptx_sm100.cuh"
#include "w8a8_device.cuh"

namespace b200q {
namespace {

constexpr int kPairBN = 256;                  // N of the pair's UMMA
constexpr int kHalfBN = kPairBN / 2;          // B rows each CTA loads
constexpr int kPairStageBytes = kTileA * kBlockK + kHalfBN * kBlockK;  // 32 KB per CTA
constexpr int kPairStages = 6;
constexpr int kPairSmem = kPairStages * kPairStageBytes + kStagingBytes + kScaleSmemBytes + kCtrlBytes;
constexpr int kPairTmemCols = 512;            // 2 accumulator buffers x 256 columns

struct PairParams {
  int M, N, K;
  int tiles_a2;   // ceil(M / 256): row tiles of the pair
  int tiles_b;    // ceil(N / 256)
  int k_blocks;
  const float* a_scales;
  const float* w_scales;
  const void* bias;
  void* out;
  int* status;
  int debug_flags;  // test-only: 1 = skip epilogue work, 4 = skip the global stores
};

// Row-parallel layers at prefill size: instead of its own output matrix, the SCATTER kernel
// writes every 128 x 256 partial tile into the staging area of the rank that owns those token
// rows (rank o owns rows [o * M / world, (o + 1) * M / world)), slot `rank`, with the same
// 16-byte stores — over NVLink when the owner is a peer.  The transfer of the reduce-scatter
// half of the all-reduce thus runs under the GEMM's main loop.  Nothing is signalled from
// inside the kernel: its completion (stream order) is what tp_reduce_gather_kernel
// (tp_allreduce.cu) announces to the peers.  (Per-tile flags raised behind a system fence
// were measured too: the fences stalled the epilogue, 40-50 us against 30 us per GEMM.)
struct ScatterParams {
  void* stage[8];            // every rank's staging area: [src rank][M / world][N] values
  int rank, world;
  int rows_per_owner;        // M / world, a multiple of 256
};

// Order in which a pair walks the 256-row tiles.  Plain kernel: top to bottom.  SCATTER: the
// owners take turns (starting with a different one on every rank), so that the pushes over
// NVLink are spread over the whole kernel and over all links instead of coming in one burst
// per owner.
template <bool SCATTER>
__device__ __forceinline__ int row_tile_of(int i, int tiles_a2, const ScatterParams& sp) {
  if (!SCATTER) return i;
  const int per_owner = tiles_a2 / sp.world;
  const int owner = (i + sp.rank) % sp.world;
  return owner * per_owner + i / sp.world;
}

template <typename OutT, bool SCATTER>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
w8a8_umma_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                      const __grid_constant__ CUtensorMap tmap_b, const PairParams pp,
                      const ScatterParams sp) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* staging = smem + kPairStages * kPairStageBytes;
  float* s_ws = reinterpret_cast<float*>(staging + kStagingBytes);
  uint8_t* ctrl = reinterpret_cast<uint8_t*>(s_ws) + kScaleSmemBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* tfull_bar = empty_bar + kMaxStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();  // 0 = leader of the pair
  const uint32_t smem_base = ptx::smem_u32(smem);
  const bool aligned = (smem_base & 1023u) == 0u;

  // The epilogue helpers take the single-CTA kernel's parameter block.
  KernelParams p{};
  p.rows_a = pp.M;
  p.rows_b = pp.N;
  p.bn = kPairBN;
  p.swap = 0;
  p.n_channels = pp.N;
  p.n_tokens = pp.M;
  p.a_scales = pp.a_scales;
  p.w_scales = pp.w_scales;
  p.bias = pp.bias;
  p.out = pp.out;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(full_bar + s), 1);
      ptx::mbar_init(ptx::smem_u32(empty_bar + s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(ptx::smem_u32(tfull_bar + b), 1);
      ptx::mbar_init(ptx::smem_u32(tempty_bar + b), 2 * kEpiThreads);
    }
    *abort_flag = aligned ? 0 : 2;
    ptx::fence_mbar_init();
    ptx::tma_prefetch_desc(&tmap_a);
    ptx::tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), kPairTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  // both CTAs' barriers exist before either CTA signals the other
  ptx::cluster_sync_all();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // everything above overlapped the previous kernel's tail; its results are needed from here
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();

  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int total_items = pp.tiles_a2 * pp.tiles_b;
  const bool run = aligned;  // a misaligned shared window (never seen) skips all work

  if (warp == 0) {
    if (lane == 0 && run) {
      // ------------------------------------------------------ TMA producer (both CTAs)
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = pair; ok && item < total_items; item += num_pairs) {
        const int tile_b = item % pp.tiles_b;  // column tiles fastest: neighbours write one row band
        const int tile_a2 = row_tile_of<SCATTER>(item / pp.tiles_b, pp.tiles_a2, sp);
        const int row_a = (tile_a2 * 2 + static_cast<int>(rank)) * kTileA;
        const int row_b = tile_b * kPairBN + static_cast<int>(rank) * kHalfBN;
        for (int kb = 0; kb < pp.k_blocks; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(empty_bar + stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t own_bar = ptx::smem_u32(full_bar + stage);
          const uint32_t leader_bar = ptx::map_to_cta(own_bar, 0);
          const uint32_t sa = smem_base + stage * kPairStageBytes;
          const uint32_t sb = sa + kTileA * kBlockK;
          // the leader expects the bytes of both CTAs on its barrier
          if (rank == 0) ptx::mbar_arrive_expect_tx(own_bar, 2 * kPairStageBytes);
          ptx::tma_load_2d_pair(sa, &tmap_a, leader_bar, kb * kBlockK, row_a);
          ptx::tma_load_2d_pair(sb, &tmap_b, leader_bar, kb * kBlockK, row_b);
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0 && run) {
      // ------------------------------------------------------- UMMA issuer (leader only)
      const uint32_t idesc = ptx::umma_idesc(2u, 1u, 2 * kTileA, kPairBN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int item = pair; ok && item < total_items; item += num_pairs, ++it) {
        const int buf = it & 1;
        const uint32_t tphase = static_cast<uint32_t>(it >> 1) & 1u;
        if (!ptx::mbar_wait(ptx::smem_u32(tempty_bar + buf), tphase ^ 1u, abort_flag)) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * kPairBN);
        for (int kb = 0; kb < pp.k_blocks; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(full_bar + stage), phase, abort_flag)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * kPairStageBytes;
          const uint32_t sb = sa + kTileA * kBlockK;
          const uint64_t a_desc = ptx::umma_desc_k_sw128(sa);
          const uint64_t b_desc = ptx::umma_desc_k_sw128(sb);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k)
            ptx::umma_i8_ss_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc,
                                 (kb > 0 || k > 0) ? 1u : 0u);
          // free the stage in both CTAs
          const uint32_t eb = ptx::smem_u32(empty_bar + stage);
          ptx::umma_commit_pair(eb);
          ptx::umma_commit_pair(ptx::map_to_cta(eb, 1));
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          const uint32_t tb = ptx::smem_u32(tfull_bar + buf);
          ptx::umma_commit_pair(tb);
          ptx::umma_commit_pair(ptx::map_to_cta(tb, 1));
        }
      }
    }
  } else if (run) {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int epi_warp = warp - 2;
    const int quarter = warp & 3;
    const int half = epi_warp >> 2;
    const int row_in_tile = quarter * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    uint8_t* slab = staging + epi_warp * kSlabBytes;
    const uint32_t leader_tempty0 = ptx::map_to_cta(ptx::smem_u32(tempty_bar), 0);
    int it = 0;
    for (int item = pair; item < total_items; item += num_pairs, ++it) {
      const int tile_b = item % pp.tiles_b;
      const int tile_a2 = row_tile_of<SCATTER>(item / pp.tiles_b, pp.tiles_a2, sp);
      const int tile_a = tile_a2 * 2 + static_cast<int>(rank);
      const int buf = it & 1;
      const uint32_t tphase = static_cast<uint32_t>(it >> 1) & 1u;
      float* ws_tile = s_ws + buf * 256;
      {
        const int col = tile_b * kPairBN + epi_tid;
        ws_tile[epi_tid] = col < pp.N ? __ldg(pp.w_scales + col) : 0.f;
      }
      const int row = tile_a * kTileA + row_in_tile;
      const float a_s = row < pp.M ? __ldg(pp.a_scales + row) : 0.f;
      if (SCATTER) {
        // this tile's rows belong to one owner: redirect the output there
        const int owner = (tile_a * kTileA) / sp.rows_per_owner;
        p.out = reinterpret_cast<OutT*>(sp.stage[owner]) +
                static_cast<ptrdiff_t>(sp.rank - owner) * sp.rows_per_owner * pp.N;
      }
      ptx::named_bar_sync(2, kEpiThreads);
      if (!ptx::mbar_wait(ptx::smem_u32(tfull_bar + buf), tphase, abort_flag)) break;
      ptx::tc_fence_after_sync();
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buf * kPairBN);
      uint32_t va[32], vb[32];
      // this warp's 64-column groups: half, half + 2
      ptx::tmem_ld_32x32b_x32(taddr + half * 64, va);
      ptx::tmem_ld_32x32b_x32(taddr + half * 64 + 32, vb);
#pragma unroll 1
      for (int g = 0; g < 2; ++g) {
        const int c0 = (half + 2 * g) * 64;
        ptx::tmem_ld_wait();
        if (pp.debug_flags & 1) {
          if (g == 0) {
            ptx::tmem_ld_32x32b_x32(taddr + (half + 2) * 64, va);
            ptx::tmem_ld_32x32b_x32(taddr + (half + 2) * 64 + 32, vb);
          }
          continue;
        }
        const int row0 = tile_a * kTileA + quarter * 32;
        const int col0 = tile_b * kPairBN + c0;
        if (pp.bias != nullptr) {
          convert_chunk<OutT, true>(p, ws_tile + c0, a_s, col0, lane, 0, slab, va);
          convert_chunk<OutT, true>(p, ws_tile + c0 + 32, a_s, col0 + 32, lane, 1, slab, vb);
        } else {
          convert_chunk<OutT, false>(p, ws_tile + c0, a_s, col0, lane, 0, slab, va);
          convert_chunk<OutT, false>(p, ws_tile + c0 + 32, a_s, col0 + 32, lane, 1, slab, vb);
        }
        if (g == 0) {
          ptx::tmem_ld_32x32b_x32(taddr + (half + 2) * 64, va);
          ptx::tmem_ld_32x32b_x32(taddr + (half + 2) * 64 + 32, vb);
        }
        __syncwarp();
        if (!(pp.debug_flags & 4)) store_group<OutT>(p, slab, lane, row0, col0);
        __syncwarp();
      }
      // accumulator drained: tell the leader's UMMA issuer (local or remote arrive)
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive_cluster(leader_tempty0 + static_cast<uint32_t>(buf) * 8u);
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  ptx::tc_fence_before_sync();
  __syncthreads();
  // neither CTA may leave (or free TMEM) while its peer can still signal it
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem_base, kPairTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag != 0) {
    atomicCAS(pp.status, 0, 0x400 | (*abort_flag << 4) | (static_cast<int>(blockIdx.x) << 12));
  }
}

template <typename OutT, bool SCATTER = false>
cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const PairParams& pp,
                        int grid, cudaStream_t stream, const ScatterParams& sp = ScatterParams{}) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = w8a8_umma_pair_kernel<OutT, SCATTER>;
  if (dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  return launch_overlapped(kern, grid, kThreads, kPairSmem, stream, ta, tb, pp, sp);
}

}  // namespace

// The CTA-pair kernel takes prefill-sized problems whose output stores can use the
// full-line path; everything else stays on the single-CTA kernel.
bool umma_pair_applicable(int M, int N, int K, bool raw_int32_out) {
  if (env_int("B200Q_DEBUG_NO_PAIR", 0) != 0) return false;
  if (raw_int32_out || (N % 8) != 0 || (K % 16) != 0) return false;
  const long long pair_tiles =
      static_cast<long long>((M + 255) / 256) * ((N + kPairBN - 1) / kPairBN);
  return M >= 512 && pair_tiles >= sm_count() / 2;
}

// Scatter variant for row-parallel layers: partial tiles go to the owners' staging areas.
int launch_w8a8_umma_pair_scatter(const GemmArgs& a, void* const* peer_stage, int rank,
                                  int world) {
  CUtensorMap ta, tb;
  if (!get_tensor_map(a.x, a.M, a.K, kTileA, kBlockK, &ta)) return B200Q_ERR_LAUNCH;
  if (!get_tensor_map(a.w, a.N, a.K, kHalfBN, kBlockK, &tb)) return B200Q_ERR_LAUNCH;
  PairParams pp{};
  pp.M = a.M;
  pp.N = a.N;
  pp.K = a.K;
  pp.tiles_a2 = (a.M + 255) / 256;
  pp.tiles_b = (a.N + kPairBN - 1) / kPairBN;
  pp.k_blocks = (a.K + kBlockK - 1) / kBlockK;
  pp.a_scales = a.a_scales;
  pp.w_scales = a.w_scales;
  pp.bias = a.bias;
  pp.out = nullptr;
  pp.status = a.status;
  pp.debug_flags = 0;
  ScatterParams sp{};
  for (int r = 0; r < world; ++r) sp.stage[r] = peer_stage[r];
  sp.rank = rank;
  sp.world = world;
  sp.rows_per_owner = a.M / world;
  const long long items = static_cast<long long>(pp.tiles_a2) * pp.tiles_b;
  const int pairs = static_cast<int>(std::min<long long>(items, sm_count() / 2));
  cudaError_t e = a.dtype == B200Q_DTYPE_BF16
                      ? launch_pair<__nv_bfloat16, true>(ta, tb, pp, pairs * 2, a.stream, sp)
                      : launch_pair<__half, true>(ta, tb, pp, pairs * 2, a.stream, sp);
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch();
  return B200Q_OK;
}

int launch_w8a8_umma_pair(const GemmArgs& a) {
  CUtensorMap ta, tb;
  if (!get_tensor_map(a.x, a.M, a.K, kTileA, kBlockK, &ta)) return B200Q_ERR_LAUNCH;
  if (!get_tensor_map(a.w, a.N, a.K, kHalfBN, kBlockK, &tb)) return B200Q_ERR_LAUNCH;
  PairParams pp{};
  pp.M = a.M;
  pp.N = a.N;
  pp.K = a.K;
  pp.tiles_a2 = (a.M + 255) / 256;
  pp.tiles_b = (a.N + kPairBN - 1) / kPairBN;
  pp.k_blocks = (a.K + kBlockK - 1) / kBlockK;
  pp.a_scales = a.a_scales;
  pp.w_scales = a.w_scales;
  pp.bias = a.bias;
  pp.out = a.y;
  pp.status = a.status;
  pp.debug_flags = env_int("B200Q_DEBUG_FLAGS", 0);
  const long long items = static_cast<long long>(pp.tiles_a2) * pp.tiles_b;
  const int pairs = static_cast<int>(std::min<long long>(items, sm_count() / 2));
  cudaError_t e = a.dtype == B200Q_DTYPE_BF16
                      ? launch_pair<__nv_bfloat16>(ta, tb, pp, pairs * 2, a.stream)
                      : launch_pair<__half>(ta, tb, pp, pairs * 2, a.stream);
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch();
  return B200Q_OK;
}

}  // namespace b200q
