// Prefill GEMMs on CTA pairs: tcgen05.mma.cta_group::2, 256 x 256 output tile per pair.
//
// Two CTAs on neighbouring SMs (a cluster of two) share one UMMA: each CTA loads its own
// 128 token rows of A and HALF of the 256 weight rows of B per K block (32 KB instead of
// the 48 KB a single-CTA 128 x 256 tile needs), the leader CTA issues the MMAs for both,
// and each CTA finds its 128 x 256 accumulator in its own TMEM.
//
// One kernel template serves three contractions (K block = 128 bytes of a row in all of them):
//   W8A8          int8 x int8 -> int32 (kind::i8), epilogue (float(acc) * a_s[m]) * w_s[n] + b[n]
//                 (nanovllm/quantization/csrc/w8a8_gemm.cu:165-183, 387-390)
//   W8A8 raw      the same accumulators written out as int32 (parity checks)
//   W8A16         16-bit x 16-bit -> fp32 (kind::f16) on weights that w8a16_expand_kernel has
//                 expanded from int8 ONCE per call into the caller's workspace (exact: every
//                 int8 code is representable), epilogue acc * s[n] + b[n]
//                 (nanovllm/quantization/csrc/int8_weight_only_gemm.cu:397-412 expands per tile)
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
// Output routes of the epilogue (eight warps, two per TMEM lane quarter):
//   EPI_TMA     convert -> swizzled shared-memory slab -> one thread issues a TMA tensor store
//               of the 32 x 64 box (this GPU's memory only); the epilogue warps never read the
//               slab back and never issue a global store, and the stores drain while the next
//               64 columns are converted (two slabs per warp).
//   EPI_LSU     convert -> slab -> the warp reads it back row-wise and stores full 128-byte
//               lines with st.global (the only route that may write to a peer GPU: SCATTER).
//   EPI_DIRECT  raw int32 accumulators only: each thread writes its 128-byte row pieces from
//               registers.  (For 16-bit outputs this route was measured too: 32-byte stores
//               from registers need no shared memory but cost 36.1 us against 33.4 for the
//               1024 -> 4096 projection at 8192 tokens.)
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "common.h"
#include "ptx_sm100.cuh"

namespace b200q {
namespace {

constexpr int kTileRows = 128;                // rows of A (and of B) each CTA loads per K block
constexpr int kBlockBytes = 128;              // bytes of K per pipeline stage = one swizzle row
constexpr int kUmmaBytes = 32;                // bytes of K per tcgen05.mma (32 int8 / 16 halves)
constexpr int kPairBN = 256;                  // N of the pair's UMMA
constexpr int kStageBytes = 2 * kTileRows * kBlockBytes;  // 32 KB per CTA
constexpr int kEpiWarps = 8;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kThreads = 64 + kEpiThreads;    // + warp 0 (TMA) + warp 1 (UMMA)
constexpr int kSlabBytes = 32 * 128;          // 32 rows x 64 columns x 2 bytes
constexpr int kScaleBytes = 2 * 256 * 4;      // channel scales of two tiles in flight
constexpr int kCtrlBytes = 256;
constexpr int kTmemCols = 512;                // 2 accumulator buffers x 256 columns
constexpr int kMaxPairStages = 7;

enum { KIND_I8 = 0, KIND_I8_RAW = 1, KIND_F16 = 2 };
enum { EPI_LSU = 0, EPI_TMA = 1, EPI_DIRECT = 2 };

template <int EPI>
struct Shape {
  static constexpr int kSlabs = EPI == EPI_TMA ? 2 : (EPI == EPI_LSU ? 1 : 0);  // per warp
  static constexpr int kStages = EPI == EPI_TMA ? 5 : (EPI == EPI_LSU ? 6 : 7);
  static constexpr int kStagingBytes = kEpiWarps * kSlabs * kSlabBytes;
  static constexpr int kSmem = kStages * kStageBytes + kStagingBytes + kScaleBytes + kCtrlBytes;
  static_assert(kSmem <= 227 * 1024, "shared memory budget");
};

struct PairParams {
  int M, N;
  int tiles_m2;   // ceil(M / 256): row tiles of the pair
  int tiles_n;    // ceil(N / 256)
  int k_blocks;
  int m_fastest;  // order of the tile walk: 1 = neighbouring items share the weight tile
  const float* a_scales;  // per token (W8A8)
  const float* w_scales;  // per channel
  const void* bias;       // per channel, OutT, or nullptr
  void* out;              // OutT [M, N] (int32 [M, N] for KIND_I8_RAW)
  int* status;
  uint32_t idesc;         // instruction descriptor (operand and accumulator formats)
  int debug_flags;        // test hook: 1 = skip epilogue arithmetic, 4 = skip the output stores
};

// Row-parallel layers at prefill size: instead of its own output matrix, the SCATTER kernel
// writes every 128 x 256 partial tile into the staging area of the rank that owns those token
// rows (rank o owns rows [o * M / world, (o + 1) * M / world)), slot `rank`, with 16-byte
// stores — over NVLink when the owner is a peer.  The transfer of the reduce-scatter
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
__device__ __forceinline__ int row_tile_of(int i, int tiles_m2, const ScatterParams& sp) {
  if (!SCATTER) return i;
  const int per_owner = tiles_m2 / sp.world;
  const int owner = (i + sp.rank) % sp.world;
  return owner * per_owner + i / sp.world;
}

// Tile walk.  The CTA pairs work on about 74 consecutive items at a time, so the operand that
// changes slowest along the walk is re-read from L2 by neighbouring pairs while the other one
// streams.  Column tiles fastest (neighbours share token rows and write one row band) unless
// the weights are the larger operand: then row tiles go fastest, so that each weight tile is
// fetched from HBM once instead of once per 256-row band (4096 -> 24576 at 8192 tokens, 16-bit
// weights of 201 MB against a 126 MB L2: 1554 us before, against 1208 us for the library GEMM).
template <bool SCATTER>
__device__ __forceinline__ void item_to_tile(int item, const PairParams& pp, const ScatterParams& sp,
                                             int* tile_n, int* tile_m2) {
  if (!SCATTER && pp.m_fastest) {
    *tile_n = item / pp.tiles_m2;
    *tile_m2 = item - *tile_n * pp.tiles_m2;
  } else {
    *tile_n = item % pp.tiles_n;
    *tile_m2 = row_tile_of<SCATTER>(item / pp.tiles_n, pp.tiles_m2, sp);
  }
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
  const __nv_bfloat162 h = __float22bfloat162_rn(v);  // one cvt.rn.bf16x2.f32
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2_rn<__half>(float2 v) {
  const __half2 h = __float22half2_rn(v);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// 32 accumulators of one row -> 16 packed 16-bit pairs.  Packed fp32x2 arithmetic (mul.f32x2
// rounds each half like the scalar instruction, so results equal the scalar formula):
//   W8A8 : (float(acc) * a_s) * w_s [+ bias]      W8A16: acc * w_s [+ bias]
template <int KIND, typename OutT, bool HAS_BIAS>
__device__ __forceinline__ void convert32(const float* s_ws, float a_s, const OutT* bias, int col0,
                                          int n_cols, const uint32_t (&v)[32],
                                          uint32_t (&packed)[16]) {
  const float2 a2 = make_float2(a_s, a_s);
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 ws = *reinterpret_cast<const float4*>(s_ws + j);
    float2 lo, hi;
    if (KIND == KIND_F16) {
      lo = __fmul2_rn(make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1])),
                      make_float2(ws.x, ws.y));
      hi = __fmul2_rn(make_float2(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])),
                      make_float2(ws.z, ws.w));
    } else {
      lo = make_float2(static_cast<float>(static_cast<int>(v[j])),
                       static_cast<float>(static_cast<int>(v[j + 1])));
      hi = make_float2(static_cast<float>(static_cast<int>(v[j + 2])),
                       static_cast<float>(static_cast<int>(v[j + 3])));
      lo = __fmul2_rn(__fmul2_rn(lo, a2), make_float2(ws.x, ws.y));
      hi = __fmul2_rn(__fmul2_rn(hi, a2), make_float2(ws.z, ws.w));
    }
    if (HAS_BIAS) {
      float b[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        b[u] = col0 + j + u < n_cols ? to_float<OutT>(bias[col0 + j + u]) : 0.f;
      // scalar adds: __fadd_rn is never contracted with the multiply before it (the
      // packed add was seen fused into an fma.f32x2, one rounding instead of two)
      lo = make_float2(__fadd_rn(lo.x, b[0]), __fadd_rn(lo.y, b[1]));
      hi = make_float2(__fadd_rn(hi.x, b[2]), __fadd_rn(hi.y, b[3]));
    }
    packed[j / 2] = pack2_rn<OutT>(lo);
    packed[j / 2 + 1] = pack2_rn<OutT>(hi);
  }
}

// Parks 32 converted columns in this thread's row of a slab: rows of 128 bytes, 16-byte chunk
// c of row r stored at chunk c ^ (r & 7) — the 128-byte swizzle of a TMA box, and free of
// bank conflicts for both the row-wise writes and the reads of store_slab_rows().
__device__ __forceinline__ void park32(uint8_t* slab, int lane, int chunk_half,
                                       const uint32_t (&packed)[16]) {
  const int sw = lane & 7;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int chunk = chunk_half * 4 + c;
    *reinterpret_cast<uint4*>(slab + lane * 128 + ((chunk ^ sw) << 4)) =
        make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
  }
}

// EPI_LSU: reads the warp's 32 x 64 slab back row-wise (8 lanes per 128-byte row) and stores
// full rows: every store instruction writes four complete 128-byte lines.
template <typename OutT>
__device__ __forceinline__ void store_slab_rows(OutT* out, int M, int N, const uint8_t* slab,
                                                int lane, int row0, int col0) {
  const int c = lane & 7;
  const int col = col0 + c * 8;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3);
    const uint4 val = *reinterpret_cast<const uint4*>(slab + r * 128 + ((c ^ (r & 7)) << 4));
    const int row = row0 + r;
    if (row < M && col < N)  // N % 8 == 0: a 16-byte piece is all in or all out
      *reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * N + col) = val;
  }
}

// Raw accumulators: 32 int32 (one 128-byte line when N % 32 == 0) per thread.
__device__ __forceinline__ void store_row_i32(int32_t* out, int M, int N, int row, int col0,
                                              const uint32_t (&v)[32]) {
  if (row >= M || col0 >= N) return;
  int32_t* dst = out + static_cast<size_t>(row) * N + col0;
  if (col0 + 32 <= N && (N & 3) == 0) {
#pragma unroll
    for (int j = 0; j < 32; j += 4)
      *reinterpret_cast<uint4*>(dst + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < N) dst[j] = static_cast<int32_t>(v[j]);
  }
}

template <int KIND, typename OutT, int EPI, bool SCATTER>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
umma_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_y, const PairParams pp,
                 const ScatterParams sp) {
  using S = Shape<EPI>;
  constexpr int kStages = S::kStages;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* staging = smem + kStages * kStageBytes;
  float* s_ws = reinterpret_cast<float*>(staging + S::kStagingBytes);
  uint8_t* ctrl = reinterpret_cast<uint8_t*>(s_ws) + kScaleBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + kMaxPairStages;
  uint64_t* tfull_bar = empty_bar + kMaxPairStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();  // 0 = leader of the pair
  const uint32_t smem_base = ptx::smem_u32(smem);
  const bool aligned = (smem_base & 1023u) == 0u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
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
    if (EPI == EPI_TMA) ptx::tma_prefetch_desc(&tmap_y);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  // both CTAs' barriers exist before either CTA signals the other
  ptx::cluster_sync_all();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int total_items = pp.tiles_m2 * pp.tiles_n;
  // Weights do not depend on the previous kernel: ask L2 for this CTA's first weight rows while
  // that kernel is still running (a prefetch is only a hint, so it is safe even if they did).
  if (KIND != KIND_F16 && threadIdx.x == 0 && aligned && pair < total_items) {
    const int first_n = pp.m_fastest ? pair / pp.tiles_m2 : pair % pp.tiles_n;
    const int row_b = first_n * kPairBN + static_cast<int>(rank) * kTileRows;
    const int n = pp.k_blocks < 8 ? pp.k_blocks : 8;
    for (int kb = 0; kb < n; ++kb) ptx::tma_prefetch_l2_2d(&tmap_b, kb * kBlockBytes, row_b);
  }
  // everything above overlapped the previous kernel's tail; its results are needed from here
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();

  const bool run = aligned;  // a misaligned shared window (never seen) skips all work

  if (warp == 0) {
    if (lane == 0 && run) {
      // ------------------------------------------------------ TMA producer (both CTAs)
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = pair; ok && item < total_items; item += num_pairs) {
        int tile_n, tile_m2;
        item_to_tile<SCATTER>(item, pp, sp, &tile_n, &tile_m2);
        const int row_a = (tile_m2 * 2 + static_cast<int>(rank)) * kTileRows;
        const int row_b = tile_n * kPairBN + static_cast<int>(rank) * kTileRows;
        for (int kb = 0; kb < pp.k_blocks; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(empty_bar + stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t own_bar = ptx::smem_u32(full_bar + stage);
          const uint32_t leader_bar = ptx::map_to_cta(own_bar, 0);
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kTileRows * kBlockBytes;
          // the leader expects the bytes of both CTAs on its barrier
          if (rank == 0) ptx::mbar_arrive_expect_tx(own_bar, 2 * kStageBytes);
          ptx::tma_load_2d_pair(sa, &tmap_a, leader_bar, kb * kBlockBytes, row_a);
          ptx::tma_load_2d_pair(sb, &tmap_b, leader_bar, kb * kBlockBytes, row_b);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0 && run) {
      // ------------------------------------------------------- UMMA issuer (leader only)
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
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kTileRows * kBlockBytes;
          const uint64_t a_desc = ptx::umma_desc_k_sw128(sa);
          const uint64_t b_desc = ptx::umma_desc_k_sw128(sb);
#pragma unroll
          for (int k = 0; k < kBlockBytes / kUmmaBytes; ++k) {
            const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
            if (pp.debug_flags & 2) continue;  // test hook: time the pipeline without the MMAs
            if (KIND == KIND_F16)
              ptx::umma_f16_ss_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, pp.idesc, acc);
            else
              ptx::umma_i8_ss_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, pp.idesc, acc);
          }
          // free the stage in both CTAs (one commit, signal delivered to both)
          ptx::umma_commit_pair_both(ptx::smem_u32(empty_bar + stage));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) ptx::umma_commit_pair_both(ptx::smem_u32(tfull_bar + buf));
      }
    }
  } else if (run) {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int epi_warp = warp - 2;
    const int quarter = warp & 3;      // the TMEM lane quarter this warp may read
    const int half = epi_warp >> 2;    // this warp's 64-column groups: half, half + 2
    const int row_in_tile = quarter * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    uint8_t* slabs = staging + epi_warp * (S::kSlabs * kSlabBytes);
    const uint32_t leader_tempty0 = ptx::map_to_cta(ptx::smem_u32(tempty_bar), 0);
    const OutT* bias = reinterpret_cast<const OutT*>(pp.bias);
    int it = 0;
    for (int item = pair; item < total_items; item += num_pairs, ++it) {
      int tile_n, tile_m2;
      item_to_tile<SCATTER>(item, pp, sp, &tile_n, &tile_m2);
      const int tile_m = tile_m2 * 2 + static_cast<int>(rank);
      const int buf = it & 1;
      const uint32_t tphase = static_cast<uint32_t>(it >> 1) & 1u;
      float* ws_tile = s_ws + buf * 256;
      if (KIND != KIND_I8_RAW) {
        const int col = tile_n * kPairBN + epi_tid;
        ws_tile[epi_tid] = col < pp.N ? __ldg(pp.w_scales + col) : 0.f;
      }
      const int row = tile_m * kTileRows + row_in_tile;
      const float a_s = (KIND == KIND_I8 && row < pp.M) ? __ldg(pp.a_scales + row) : 0.f;
      OutT* out = reinterpret_cast<OutT*>(pp.out);
      if (SCATTER) {
        // this tile's rows belong to one owner: redirect the output there
        const int owner = (tile_m * kTileRows) / sp.rows_per_owner;
        out = reinterpret_cast<OutT*>(sp.stage[owner]) +
              static_cast<ptrdiff_t>(sp.rank - owner) * sp.rows_per_owner * pp.N;
      }
      ptx::named_bar_sync(2, kEpiThreads);
      if (!ptx::mbar_wait(ptx::smem_u32(tfull_bar + buf), tphase, abort_flag)) break;
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(buf * kPairBN);
      uint32_t va[32], vb[32];
      ptx::tmem_ld_32x32b_x32(taddr + half * 64, va);
      ptx::tmem_ld_32x32b_x32(taddr + half * 64 + 32, vb);
#pragma unroll 1
      for (int g = 0; g < 2; ++g) {
        const int c0 = (half + 2 * g) * 64;
        const int row0 = tile_m * kTileRows + quarter * 32;
        const int col0 = tile_n * kPairBN + c0;
        ptx::tmem_ld_wait();
        if (KIND == KIND_I8_RAW) {
          if (!(pp.debug_flags & 4)) {
            store_row_i32(reinterpret_cast<int32_t*>(pp.out), pp.M, pp.N, row, col0, va);
            store_row_i32(reinterpret_cast<int32_t*>(pp.out), pp.M, pp.N, row, col0 + 32, vb);
          }
          if (g == 0) {
            ptx::tmem_ld_32x32b_x32(taddr + (half + 2) * 64, va);
            ptx::tmem_ld_32x32b_x32(taddr + (half + 2) * 64 + 32, vb);
          }
          continue;
        }
        if (pp.debug_flags & 1) {
          if (g == 0) {
            ptx::tmem_ld_32x32b_x32(taddr + (half + 2) * 64, va);
            ptx::tmem_ld_32x32b_x32(taddr + (half + 2) * 64 + 32, vb);
          }
          continue;
        }
        uint32_t pa[16], pb[16];
        if (bias != nullptr) {
          convert32<KIND, OutT, true>(ws_tile + c0, a_s, bias, col0, pp.N, va, pa);
          convert32<KIND, OutT, true>(ws_tile + c0 + 32, a_s, bias, col0 + 32, pp.N, vb, pb);
        } else {
          convert32<KIND, OutT, false>(ws_tile + c0, a_s, bias, col0, pp.N, va, pa);
          convert32<KIND, OutT, false>(ws_tile + c0 + 32, a_s, bias, col0 + 32, pp.N, vb, pb);
        }
        if (g == 0) {
          ptx::tmem_ld_32x32b_x32(taddr + (half + 2) * 64, va);
          ptx::tmem_ld_32x32b_x32(taddr + (half + 2) * 64 + 32, vb);
        }
        if (EPI == EPI_DIRECT) {
          // raw accumulators only (handled above)
        } else if (EPI == EPI_TMA) {
          uint8_t* slab = slabs + g * kSlabBytes;
          // the store issued from this slab one tile ago must have finished reading it;
          // the one issued since (other slab) may still be running
          if (lane == 0) ptx::bulk_wait_group_read<1>();
          __syncwarp();
          park32(slab, lane, 0, pa);
          park32(slab, lane, 1, pb);
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (!(pp.debug_flags & 4) && row0 < pp.M && col0 < pp.N)
              ptx::tma_store_2d(&tmap_y, ptx::smem_u32(slab), col0 * 2, row0);
            ptx::bulk_commit_group();  // always: the wait above counts groups
          }
        } else {
          uint8_t* slab = slabs;
          park32(slab, lane, 0, pa);
          park32(slab, lane, 1, pb);
          __syncwarp();
          if (!(pp.debug_flags & 4)) store_slab_rows<OutT>(out, pp.M, pp.N, slab, lane, row0, col0);
          __syncwarp();
        }
      }
      // accumulator drained: tell the leader's UMMA issuer (local or remote arrive)
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive_cluster(leader_tempty0 + static_cast<uint32_t>(buf) * 8u);
    }
    // shared memory must stay valid until the last TMA store has read it, and the output
    // must be complete when the kernel ends
    if (EPI == EPI_TMA && lane == 0) ptx::bulk_wait_group<0>();
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  ptx::tc_fence_before_sync();
  __syncthreads();
  // neither CTA may leave (or free TMEM) while its peer can still signal it
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag != 0) {
    atomicCAS(pp.status, 0, 0x400 | (*abort_flag << 4) | (static_cast<int>(blockIdx.x) << 12));
  }
}

// Four int8 (one word) -> four values of type T (two words), exact, without integer-to-float
// conversions: fp16: 0x6400 | u is the half 1024 + u (u = q + 128), minus 1152; bf16:
// 0x4B000000 | u is the float 2^23 + u, minus 2^23 + 128, and the upper half of that fp32
// word (an integer of at most 8 significant bits) is its bf16 form.
template <typename T>
__device__ __forceinline__ uint2 expand_word(uint32_t w);
template <>
__device__ __forceinline__ uint2 expand_word<__half>(uint32_t w) {
  const uint32_t t = w ^ 0x80808080u;
  uint32_t lo = __byte_perm(t, 0x64646464u, 0x4140);
  uint32_t hi = __byte_perm(t, 0x64646464u, 0x4342);
  const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
  const __half2 l = __hsub2(*reinterpret_cast<__half2*>(&lo), bias);
  const __half2 h = __hsub2(*reinterpret_cast<__half2*>(&hi), bias);
  return make_uint2(*reinterpret_cast<const uint32_t*>(&l), *reinterpret_cast<const uint32_t*>(&h));
}
template <>
__device__ __forceinline__ uint2 expand_word<__nv_bfloat16>(uint32_t w) {
  const uint32_t t = w ^ 0x80808080u;
  const float2 m = make_float2(-8388736.f, -8388736.f);
  const float2 f01 = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(t, 0x4B000000u, 0x7540)),
                                            __uint_as_float(__byte_perm(t, 0x4B000000u, 0x7541))), m);
  const float2 f23 = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(t, 0x4B000000u, 0x7542)),
                                            __uint_as_float(__byte_perm(t, 0x4B000000u, 0x7543))), m);
  return make_uint2(__byte_perm(__float_as_uint(f01.x), __float_as_uint(f01.y), 0x7632),
                    __byte_perm(__float_as_uint(f23.x), __float_as_uint(f23.y), 0x7632));
}

// int8 [n] -> T [n], exact (|q| <= 128 has at most 8 significant bits).  16 codes per thread.
template <typename T>
__global__ void __launch_bounds__(256) w8a16_expand_kernel(const int8_t* __restrict__ q,
                                                           T* __restrict__ out, size_t n16) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride) {
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(q) + i);
    const uint2 e0 = expand_word<T>(w.x), e1 = expand_word<T>(w.y), e2 = expand_word<T>(w.z),
                e3 = expand_word<T>(w.w);
    uint4* dst = reinterpret_cast<uint4*>(out) + 2 * i;
    dst[0] = make_uint4(e0.x, e0.y, e1.x, e1.y);
    dst[1] = make_uint4(e2.x, e2.y, e3.x, e3.y);
  }
}

template <int KIND, typename OutT, int EPI, bool SCATTER = false>
cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& ty,
                        const PairParams& pp, int grid, cudaStream_t stream,
                        const ScatterParams& sp = ScatterParams{}) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = umma_pair_kernel<KIND, OutT, EPI, SCATTER>;
  constexpr int smem = Shape<EPI>::kSmem;
  if (dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  return launch_overlapped(kern, grid, kThreads, smem, stream, ta, tb, ty, pp, sp);
}

template <int KIND, typename OutT>
cudaError_t launch_pair_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb,
                            const CUtensorMap& ty, const PairParams& pp, int grid,
                            cudaStream_t stream) {
  switch (epi) {
    case EPI_LSU:
      return launch_pair<KIND, OutT, EPI_LSU>(ta, tb, ty, pp, grid, stream);
    default:
      return launch_pair<KIND, OutT, EPI_TMA>(ta, tb, ty, pp, grid, stream);
  }
}

PairParams make_params(const GemmArgs& a, int k_bytes) {
  PairParams pp{};
  pp.M = a.M;
  pp.N = a.N;
  pp.tiles_m2 = (a.M + 255) / 256;
  pp.tiles_n = (a.N + kPairBN - 1) / kPairBN;
  pp.k_blocks = (k_bytes + kBlockBytes - 1) / kBlockBytes;
  pp.a_scales = a.a_scales;
  pp.w_scales = a.w_scales;
  pp.bias = a.bias;
  pp.out = a.y;
  pp.status = a.status;
  pp.debug_flags = debug_knob(B200Q_KNOB_FLAGS, 0);
  pp.m_fastest = a.N > a.M ? 1 : 0;
  return pp;
}

int pair_grid(const PairParams& pp) {
  const long long items = static_cast<long long>(pp.tiles_m2) * pp.tiles_n;
  return 2 * static_cast<int>(std::min<long long>(items, sm_count() / 2));
}

// Tiles of 256 x 256 the problem has, against the number a kernel needs to be worth taking
// (default: one per CTA pair of the device).
bool enough_pair_tiles(int M, int N, int dflt_min) {
  const long long pair_tiles =
      static_cast<long long>((M + 255) / 256) * ((N + kPairBN - 1) / kPairBN);
  return pair_tiles >= debug_knob(B200Q_KNOB_PAIR_MIN_TILES, dflt_min);
}

int finish(cudaError_t e, int launches = 1) {
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch(launches);
  return B200Q_OK;
}

}  // namespace

// The CTA-pair kernel takes prefill-sized problems whose output rows are 16-byte multiples;
// everything else stays on the single-CTA kernel.  Thresholds from graph-replayed launches of
// the Qwen3-0.6B / 8B projections and their tensor-parallel shards at 512-8192 tokens: with one
// tile per CTA pair or more the pair kernel wins (1024 -> 6144 at 1024 tokens, 96 tiles: 11.6
// against 13.1 us); with fewer it wins only where the K loop is long (12288 -> 4096 at 1024
// tokens, 64 tiles: 37.0 against 40.4 us; 2048 -> 1024 at 4096 tokens, 64 tiles: 11.4 against
// 10.8 us the other way).
bool umma_pair_applicable(int M, int N, int K, bool raw_int32_out) {
  if (debug_knob(B200Q_KNOB_NO_PAIR, 0) != 0) return false;
  if ((K % 16) != 0 || M < 512) return false;
  if (!raw_int32_out && (N % 8) != 0) return false;
  const int pairs = sm_count() / 2;
  return enough_pair_tiles(M, N, K >= 4096 ? (pairs * 2) / 3 : pairs);
}

// Scatter variant for row-parallel layers: partial tiles go to the owners' staging areas.
int launch_w8a8_umma_pair_scatter(const GemmArgs& a, void* const* peer_stage, int rank,
                                  int world) {
  CUtensorMap ta, tb;
  if (!make_tensor_map(a.x, a.M, a.K, kTileRows, kBlockBytes, &ta)) return B200Q_ERR_LAUNCH;
  if (!get_tensor_map(a.w, a.N, a.K, kTileRows, kBlockBytes, &tb)) return B200Q_ERR_LAUNCH;
  PairParams pp = make_params(a, a.K);
  pp.out = nullptr;
  pp.idesc = ptx::umma_idesc(2u, 1u, 2 * kTileRows, kPairBN);
  pp.debug_flags = 0;
  ScatterParams sp{};
  for (int r = 0; r < world; ++r) sp.stage[r] = peer_stage[r];
  sp.rank = rank;
  sp.world = world;
  sp.rows_per_owner = a.M / world;
  const int grid = pair_grid(pp);
  return finish(a.dtype == B200Q_DTYPE_BF16
                    ? launch_pair<KIND_I8, __nv_bfloat16, EPI_LSU, true>(ta, tb, ta, pp, grid, a.stream, sp)
                    : launch_pair<KIND_I8, __half, EPI_LSU, true>(ta, tb, ta, pp, grid, a.stream, sp));
}

int launch_w8a8_umma_pair(const GemmArgs& a) {
  CUtensorMap ta, tb, ty;
  if (!make_tensor_map(a.x, a.M, a.K, kTileRows, kBlockBytes, &ta)) return B200Q_ERR_LAUNCH;
  if (!get_tensor_map(a.w, a.N, a.K, kTileRows, kBlockBytes, &tb)) return B200Q_ERR_LAUNCH;
  PairParams pp = make_params(a, a.K);
  pp.idesc = ptx::umma_idesc(2u, 1u, 2 * kTileRows, kPairBN);
  const int grid = pair_grid(pp);
  if (a.acc_out != nullptr) {
    pp.out = a.acc_out;
    return finish(launch_pair<KIND_I8_RAW, __nv_bfloat16, EPI_DIRECT>(ta, tb, ta, pp, grid, a.stream));
  }
  // output box of the TMA store: 64 columns (128 bytes) x 32 rows, 128-byte swizzle
  if (!make_tensor_map(a.y, a.M, static_cast<uint64_t>(a.N) * 2, 32, 128, &ty)) return B200Q_ERR_LAUNCH;
  const int epi = debug_knob(B200Q_KNOB_PAIR_EPILOGUE, EPI_TMA);
  return finish(a.dtype == B200Q_DTYPE_BF16
                    ? launch_pair_epi<KIND_I8, __nv_bfloat16>(epi, ta, tb, ty, pp, grid, a.stream)
                    : launch_pair_epi<KIND_I8, __half>(epi, ta, tb, ty, pp, grid, a.stream));
}

// ------------------------------------------------------------------ W8A16, two-phase route
// Prefill-sized W8A16: the int8 weights are expanded to the activation type once per call
// (2 N K bytes of workspace, L2-resident for the shapes of one layer) and a plain 16-bit
// contraction runs on the pair kernel; the per-channel scale stays in the fp32 epilogue.
// Expanding inside the main loop instead repeats the expansion for every 128-token tile.
bool umma16_pair_applicable(int M, int N, int K) {
  if (debug_knob(B200Q_KNOB_NO_PAIR, 0) != 0) return false;
  if ((K % 16) != 0 || (N % 8) != 0) return false;
  if (M < debug_knob(B200Q_KNOB_W8A16_PAIR_MIN_M, 1024)) return false;
  // The kernels that expand inside the main loop are so much slower at prefill size that this
  // route pays off well before every CTA pair has a tile: 2048 -> 1024 at 2048 tokens (32
  // tiles) 18.8 against 23.0 us; only short K loops on few tiles go the other way (512 -> 1024
  // at 2048 tokens: 10.6 against 9.9 us).
  const int pairs = sm_count() / 2;
  return enough_pair_tiles(M, N, K >= 1024 ? (pairs * 2) / 5 : (pairs * 2) / 3);
}

// The first kCounterBytes of a workspace belong to the split-K kernels' tile counters (kept
// zero between calls); the expanded weights follow them.
size_t umma16_pair_workspace_bytes(int N, int K) {
  return kCounterBytes + static_cast<size_t>(N) * K * 2;
}

int launch_w8a16_umma_pair(const GemmArgs& a) {
  const size_t need = umma16_pair_workspace_bytes(a.N, a.K);
  if (a.workspace == nullptr || a.workspace_bytes < need) return B200Q_ERR_WORKSPACE;
  const bool bf16 = a.dtype == B200Q_DTYPE_BF16;
  void* expanded = static_cast<uint8_t*>(a.workspace) + kCounterBytes;
  const size_t n16 = static_cast<size_t>(a.N) * a.K / 16;
  const int blocks = static_cast<int>(std::min<size_t>((n16 + 255) / 256, static_cast<size_t>(sm_count()) * 8));
  if (bf16)
    w8a16_expand_kernel<__nv_bfloat16><<<blocks, 256, 0, a.stream>>>(
        a.w, static_cast<__nv_bfloat16*>(expanded), n16);
  else
    w8a16_expand_kernel<__half><<<blocks, 256, 0, a.stream>>>(a.w, static_cast<__half*>(expanded), n16);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return finish(e);

  CUtensorMap ta, tb, ty;
  const uint64_t k_bytes = static_cast<uint64_t>(a.K) * 2;
  if (!make_tensor_map(a.x, a.M, k_bytes, kTileRows, kBlockBytes, &ta)) return B200Q_ERR_LAUNCH;
  if (!make_tensor_map(expanded, a.N, k_bytes, kTileRows, kBlockBytes, &tb)) return B200Q_ERR_LAUNCH;
  if (!make_tensor_map(a.y, a.M, static_cast<uint64_t>(a.N) * 2, 32, 128, &ty)) return B200Q_ERR_LAUNCH;
  PairParams pp = make_params(a, static_cast<int>(k_bytes));
  pp.idesc = ptx::umma_idesc(1u, bf16 ? 1u : 0u, 2 * kTileRows, kPairBN);
  const int grid = pair_grid(pp);
  const int epi = debug_knob(B200Q_KNOB_PAIR_EPILOGUE, EPI_TMA);
  return finish(bf16 ? launch_pair_epi<KIND_F16, __nv_bfloat16>(epi, ta, tb, ty, pp, grid, a.stream)
                     : launch_pair_epi<KIND_F16, __half>(epi, ta, tb, ty, pp, grid, a.stream),
                2);
}

}  // namespace b200q
