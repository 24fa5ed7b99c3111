// W8A16 GEMM on the tcgen05 tensor cores: 16-bit activations x int8 weights.
//
//   y[m,n] = T( scales[n] * sum_k x[m,k] * float(q[n,k]) + bias[n] ),  fp32 accumulation
//
// The weights stay int8 in HBM and on their way into shared memory (TMA).  A group of
// converter warps expands each int8 K block to the activation type (exact: |q| <= 128)
// directly into the 128-byte-swizzled layout the UMMA descriptors expect, the tensor
// cores run tcgen05.mma kind::f16 on the expanded tile, and the per-channel scale is
// applied once in the fp32 epilogue.  The reference's fused kernel expands and scales
// per product (nanovllm/quantization/csrc/int8_weight_only_gemm.cu:397-412,
// 258-292); its Python path scales the whole matrix first (cuda.py:293-300); all three
// compute the same sum up to rounding.
//
// Warp roles (448 threads, 1 CTA per SM, persistent):
//   warp 0      TMA producer: 16-bit operand tile (128-byte swizzle) + raw int8 tile
//               (64-byte swizzle) per K block of 64 elements
//   warp 1      UMMA issuer (one thread): 4 x tcgen05.mma (K = 16) per K block
//   warps 2-5   epilogue: tcgen05.ld -> acc * s[n] + b[n] -> 16 bit -> global
//   warps 6-13  converters: raw int8 tile -> 16-bit swizzled tile (ring of 2 buffers)
//
// As in the W8A8 kernel the 128-row side of the UMMA tile holds the tokens for
// prefill-sized problems and the output channels for decode-sized ones ("swap"), where K
// is also split over CTAs; fp32 partial tiles are summed in a fixed order by the last CTA
// to arrive, so results do not depend on scheduling.
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

// 448 threads run; the bound of 512 keeps the kernel at 128 registers per thread, which is
// what four warps per scheduler can hold.
// CLUSTER: K split over a cluster of p.cluster CTAs, reduced in the leader's shared memory.
template <typename T, bool CLUSTER>
__global__ void __launch_bounds__(512, 1)
w8a16_umma_kernel(const __grid_constant__ CUtensorMap tmap_x,
                  const __grid_constant__ CUtensorMap tmap_w, const KernelParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  // rows of the 16-bit (activation) tile and of the int8 (weight) tile in one stage
  const int rows16 = p.swap ? p.bn : kTileA;
  const int rows8 = p.swap ? kTileA : p.bn;
  const uint32_t tile16_bytes = rows16 * kRow16;
  const uint32_t raw_bytes = rows8 * kRow8;
  const uint32_t stage_bytes = tile16_bytes + raw_bytes;
  const uint32_t conv_bytes = rows8 * kRow16;
  uint8_t* conv_base = smem + static_cast<size_t>(p.stages) * stage_bytes;
  float* partial = reinterpret_cast<float*>(conv_base + p.conv_bufs * conv_bytes);  // cluster leader
  uint8_t* staging = reinterpret_cast<uint8_t*>(partial) + p.partial_bytes;
  float* s_ws = reinterpret_cast<float*>(staging + kStagingBytes);
  uint8_t* ctrl = reinterpret_cast<uint8_t*>(s_ws) + kScaleSmemBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* cfull_bar = empty_bar + kMaxStages;     // [conv_bufs] converted tile ready
  uint64_t* cempty_bar = cfull_bar + kMaxConvBufs;  // [conv_bufs] converted tile consumed
  uint64_t* tfull_bar = cempty_bar + kMaxConvBufs;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* pfull_bar = tempty_bar + 2;             // cluster leader: partial tiles have arrived
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pfull_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [2]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = ptx::smem_u32(smem);
  if ((smem_base & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, 0x200);
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(full_bar + s), 1);
      ptx::mbar_init(ptx::smem_u32(empty_bar + s), 1);
    }
    for (int c = 0; c < p.conv_bufs; ++c) {
      ptx::mbar_init(ptx::smem_u32(cfull_bar + c), kConvWarps);
      ptx::mbar_init(ptx::smem_u32(cempty_bar + c), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(ptx::smem_u32(tfull_bar + b), 1);
      ptx::mbar_init(ptx::smem_u32(tempty_bar + b), kEpiThreads);
    }
    ptx::mbar_init(ptx::smem_u32(pfull_bar), static_cast<uint32_t>(max(1, p.cluster - 1) * kEpiThreads));
    *abort_flag = 0;
    last_flag[0] = 0;
    last_flag[1] = 0;
    ptx::fence_mbar_init();
    ptx::tma_prefetch_desc(&tmap_x);
    ptx::tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), static_cast<uint32_t>(p.tmem_cols));
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  // the leader's barrier and partial-tile area exist before a peer CTA writes to them
  constexpr bool clustered = CLUSTER;
  if (clustered) ptx::cluster_sync_all();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // everything above overlapped the previous kernel's tail; its results are needed from here
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();

  const int total_items = p.tiles_a * p.tiles_b * p.splits;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------ TMA producer
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const int split = item % p.splits;
        const int t = item / p.splits;
        const int tile_a = t % p.tiles_a;
        const int tile_b = t / p.tiles_a;
        // token tile / channel tile indices
        const int row16 = p.swap ? tile_b * p.bn : tile_a * kTileA;
        const int row8 = p.swap ? tile_a * kTileA : tile_b * p.bn;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(empty_bar + stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t bar = ptx::smem_u32(full_bar + stage);
          const uint32_t s16 = smem_base + stage * stage_bytes;
          const uint32_t s8 = s16 + tile16_bytes;
          ptx::mbar_arrive_expect_tx(bar, stage_bytes);
          ptx::tma_load_2d(s16, &tmap_x, bar, kb * kBlockK * 2, row16);  // byte coordinate
          ptx::tma_load_2d(s8, &tmap_w, bar, kb * kBlockK, row8);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------- UMMA issuer
      // A and B must have the same element type in kind::f16 (a bf16 x fp16 descriptor was
      // tried once and faulted), so the weights are expanded to the activation type.
      const uint32_t fmt = p.is_bf16 ? 1u : 0u;
      const uint32_t idesc = ptx::umma_idesc(1u, fmt, kTileA, static_cast<uint32_t>(p.bn));
      int stage = 0, cb = 0;
      uint32_t phase = 0, cphase = 0;
      int it = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x, ++it) {
        const int split = item % p.splits;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        const int buf = it & 1;
        const uint32_t tphase = static_cast<uint32_t>(it >> 1) & 1u;
        if (!ptx::mbar_wait(ptx::smem_u32(tempty_bar + buf), tphase ^ 1u, abort_flag)) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * p.bn);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(full_bar + stage), phase, abort_flag) ||
              !ptx::mbar_wait(ptx::smem_u32(cfull_bar + cb), cphase, abort_flag)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t s16 = smem_base + stage * stage_bytes;
          const uint32_t sconv = ptx::smem_u32(conv_base) + cb * conv_bytes;
          const uint64_t d16 = ptx::umma_desc_k_sw128(s16);
          const uint64_t dcv = ptx::umma_desc_k_sw128(sconv);
          const uint64_t a_desc = p.swap ? dcv : d16;
          const uint64_t b_desc = p.swap ? d16 : dcv;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            // 16 elements of 2 bytes = 32 bytes along K = +2 in 16-byte units
            ptx::umma_f16_ss(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc,
                             (kb > kb0 || k > 0) ? 1u : 0u);
          }
          ptx::umma_commit(ptx::smem_u32(empty_bar + stage));
          ptx::umma_commit(ptx::smem_u32(cempty_bar + cb));
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
          if (++cb == p.conv_bufs) {
            cb = 0;
            cphase ^= 1u;
          }
        }
        if (ok) ptx::umma_commit(ptx::smem_u32(tfull_bar + buf));
      }
    }
  } else if (warp >= 2 + kEpiWarps) {
    // ---------------------------------------------------------- converters
    const int ctid = threadIdx.x - (64 + kEpiThreads);
    int stage = 0, cb = 0;
    uint32_t phase = 0, cphase = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
      const int split = item % p.splits;
      const int kb0 = split * p.kb_per_split;
      const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!ptx::mbar_wait(ptx::smem_u32(full_bar + stage), phase, abort_flag) ||
            !ptx::mbar_wait(ptx::smem_u32(cempty_bar + cb), cphase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        const uint8_t* raw = smem + stage * stage_bytes + tile16_bytes;
        uint8_t* dst = conv_base + cb * conv_bytes;
        if (!(p.debug_flags & 8)) {
          if (rows8 * 4 <= kConvThreads) {
            if (ctid < rows8 * 4) expand_quarter_row<T>(raw, dst, ctid >> 2, ctid & 3);
          } else {
            for (int r = ctid; r < rows8; r += kConvThreads) expand_row<T>(raw, dst, r);
          }
        }
        ptx::fence_proxy_async_smem();  // generic-proxy writes -> visible to the UMMA reads
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(cfull_bar + cb));
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1u;
        }
        if (++cb == p.conv_bufs) {
          cb = 0;
          cphase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int epi_warp = warp - 2;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    const int n_chunks_tile = p.bn >> 5;
    const int n_groups = (n_chunks_tile + 1) >> 1;
    uint8_t* slab = staging + epi_warp * kSlabBytes;
    int it = 0;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it) {
      const int split = item % p.splits;
      const int t = item / p.splits;
      const int tile_a = t % p.tiles_a;
      const int tile_b = t / p.tiles_a;
      const int buf = it & 1;
      const uint32_t tphase = static_cast<uint32_t>(it >> 1) & 1u;
      const bool fast = p.fast_store && (p.splits == 1 || clustered);
      float* ws_tile = s_ws + buf * 256;
      if (clustered && split > 0) {
        // K split over the cluster: hand this CTA's partial tile to the leader (cluster rank
        // 0 = split 0) through its shared memory, laid out [split - 1][column][row]
        if (!ptx::mbar_wait(ptx::smem_u32(tfull_bar + buf), tphase, abort_flag)) break;
        ptx::tc_fence_after_sync();
        const uint32_t taddr_p = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                 static_cast<uint32_t>(buf * p.bn);
        const uint32_t dst0 = ptx::map_to_cta(ptx::smem_u32(partial), 0) +
                              (static_cast<uint32_t>((split - 1) * p.bn) * kTileA + row_in_tile) * 4u;
        for (int c = 0; c < n_chunks_tile; ++c) {
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(taddr_p + c * 32, v);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            ptx::st_shared_cluster_u32(dst0 + static_cast<uint32_t>(c * 32 + j) * (kTileA * 4u), v[j]);
        }
        ptx::tc_fence_before_sync();
        ptx::mbar_arrive(ptx::smem_u32(tempty_bar + buf));
        ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(pfull_bar), 0));  // release: stores first
        continue;
      }
      if (fast) {
        for (int i = epi_tid; i < p.bn; i += kEpiThreads) {
          const int col = tile_b * p.bn + i;
          ws_tile[i] = col < p.rows_b ? __ldg(p.w_scales + col) : 0.f;
        }
        ptx::named_bar_sync(2, kEpiThreads);
      }
      if (!ptx::mbar_wait(ptx::smem_u32(tfull_bar + buf), tphase, abort_flag)) break;
      if (clustered && !ptx::mbar_wait_cluster(ptx::smem_u32(pfull_bar), 0u, abort_flag)) break;
      ptx::tc_fence_after_sync();
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buf * p.bn);
      // leader of a cluster: add the peers' partial tiles, in split order (deterministic)
      auto add_partials = [&](int c0, uint32_t (&v)[32]) {
        for (int sp = 1; sp < p.cluster; ++sp) {
          const float* src = partial + static_cast<size_t>((sp - 1) * p.bn + c0) * kTileA + row_in_tile;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = __float_as_uint(__fadd_rn(__uint_as_float(v[j]), src[j * kTileA]));
        }
      };
      float* mine = nullptr;
      if (p.splits > 1 && !clustered)
        mine = p.partials + (static_cast<size_t>(t) * p.splits + split) * p.bn * kTileA + row_in_tile;

      auto consume = [&](int c0, const uint32_t (&v)[32]) {
        if (p.splits > 1 && !clustered) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            __stcg(mine + static_cast<size_t>(c0 + j) * kTileA, __uint_as_float(v[j]));
        } else {
          emit_chunk<T>(p, tile_a, tile_b, row_in_tile, c0, v);
        }
      };

      uint32_t va[32], vb[32];
      auto issue = [&](int g) {
        const int c = 2 * g;
        ptx::tmem_ld_32x32b_x32(taddr + c * 32, va);
        if (c + 1 < n_chunks_tile) ptx::tmem_ld_32x32b_x32(taddr + (c + 1) * 32, vb);
      };
      issue(0);
      for (int g = 0; g < n_groups; ++g) {
        const int c = 2 * g;
        const bool two = c + 1 < n_chunks_tile;
        ptx::tmem_ld_wait();
        if (p.debug_flags & 1) {
          if (g + 1 < n_groups) issue(g + 1);
          continue;
        }
        if (clustered) {
          add_partials(c * 32, va);
          if (two) add_partials(c * 32 + 32, vb);
        }
        if (fast) {
          const int row0 = tile_a * kTileA + quarter * 32;
          const int col0 = tile_b * p.bn + c * 32;
          if (p.bias != nullptr) {
            convert_chunk<T, true>(p, ws_tile + c * 32, col0, lane, 0, slab, va);
            if (two) convert_chunk<T, true>(p, ws_tile + c * 32 + 32, col0 + 32, lane, 1, slab, vb);
          } else {
            convert_chunk<T, false>(p, ws_tile + c * 32, col0, lane, 0, slab, va);
            if (two) convert_chunk<T, false>(p, ws_tile + c * 32 + 32, col0 + 32, lane, 1, slab, vb);
          }
          if (g + 1 < n_groups) issue(g + 1);
          __syncwarp();
          store_group<T>(p, slab, lane, row0, col0);
          __syncwarp();
        } else {
          consume(c * 32, va);
          if (two) consume(c * 32 + 32, vb);
          if (g + 1 < n_groups) issue(g + 1);
        }
      }
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(ptx::smem_u32(tempty_bar + buf));

      if (p.splits > 1 && !clustered) {
        __threadfence();
        ptx::named_bar_sync(1, kEpiThreads);
        if (epi_tid == 0) {
          const unsigned int old = atomicAdd(p.counters + t, 1u);
          const int last = (old == static_cast<unsigned int>(p.splits - 1));
          if (last) p.counters[t] = 0u;
          last_flag[it & 1] = last;
        }
        ptx::named_bar_sync(1, kEpiThreads);
        if (last_flag[it & 1]) {
          __threadfence();
          const float* base =
              p.partials + static_cast<size_t>(t) * p.splits * p.bn * kTileA + row_in_tile;
          for (int ch = 0; ch < n_chunks_tile; ++ch) {
            const int c0 = ch * 32;
            uint32_t v[32];
            float acc[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = 0.f;
            for (int s = 0; s < p.splits; ++s) {  // fixed order: deterministic sums
              const float* src = base + static_cast<size_t>(s) * p.bn * kTileA;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                acc[j] = __fadd_rn(acc[j], __ldcg(src + static_cast<size_t>(c0 + j) * kTileA));
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(acc[j]);
            emit_chunk<T>(p, tile_a, tile_b, row_in_tile, c0, v);
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  ptx::tc_fence_before_sync();
  __syncthreads();
  // no CTA of a cluster leaves while a peer may still write its shared memory or barriers
  if (clustered) ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
  if (threadIdx.x == 0 && *abort_flag != 0) {
    atomicCAS(p.status, 0, 0x300 | (static_cast<int>(blockIdx.x) << 12));
  }
}

int round_up(int v, int m) { return (v + m - 1) / m * m; }

template <typename T, bool CLUSTER>
cudaError_t launch_kernel(const CUtensorMap& tx, const CUtensorMap& tw, const KernelParams& kp,
                          const UmmaPlan& plan, cudaStream_t stream) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = w8a16_umma_kernel<T, CLUSTER>;
  if (dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  return launch_clustered(plan.cluster, true, kern, plan.grid, kThreads, plan.smem_bytes, stream, tx,
                          tw, kp);
}

}  // namespace

bool umma16_make_plan(int M, int N, int K, int swap, UmmaPlan* plan) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % 16) != 0) return false;
  UmmaPlan pl{};
  pl.swap = swap;
  pl.rows_a = swap ? N : M;
  pl.rows_b = swap ? M : N;
  const int sms = sm_count();
  pl.k_blocks = (K + kBlockK - 1) / kBlockK;
  int bn = pl.rows_b >= 256 ? 256 : round_up(pl.rows_b, 32);
  if (!swap && pl.rows_b >= 256) {
    const int ta = (pl.rows_a + kTileA - 1) / kTileA;
    double best = 1e30;
    for (int cand : {256, 128, 64}) {
      const int tiles = ta * ((pl.rows_b + cand - 1) / cand);
      const int waves = (tiles + sms - 1) / sms;
      const double cost = waves * (cand + 32.0);
      if (cost < best) {
        best = cost;
        bn = cand;
      }
    }
  }
  bn = debug_knob(B200Q_KNOB_BN, bn);
  if (bn < 32 || bn > 256 || (bn % 32) != 0) return false;
  pl.bn = bn;
  pl.tiles_a = (pl.rows_a + kTileA - 1) / kTileA;
  pl.tiles_b = (pl.rows_b + bn - 1) / bn;
  const long long tiles = static_cast<long long>(pl.tiles_a) * pl.tiles_b;
  if (tiles > 1 << 22) return false;
  // Split K over CTAs only when few tiles would each have a long K loop: handing partial
  // tiles over through global memory costs several microseconds, more than streaming a
  // few hundred KB of weights through one SM.
  int splits = 1;
  if (tiles * 2 <= sms && pl.k_blocks >= 128) {
    splits = static_cast<int>(sms / tiles);
    splits = std::min(splits, pl.k_blocks / 64);
    splits = std::min(splits, 8);
  }
  splits = debug_knob(B200Q_KNOB_SPLITS, splits);
  if (splits < 1) splits = 1;
  if (splits > pl.k_blocks) splits = pl.k_blocks;
  pl.kb_per_split = (pl.k_blocks + splits - 1) / splits;
  pl.splits = (pl.k_blocks + pl.kb_per_split - 1) / pl.kb_per_split;
  // Few tiles with a long K loop (decode batches of 64-512 tokens on the narrow projections):
  // a cluster of 2 or 4 CTAs splits K and the leader adds the peers' partial tiles from its own
  // shared memory — no trip through global memory, unlike the split above.
  pl.cluster = 1;
  pl.partial_bytes = 0;
  if (!swap && pl.splits == 1 && (N % 8) == 0 && (bn % 64) == 0) {
    int cl = 1;
    for (int cand : {4, 2})
      if (tiles * cand <= sms && pl.k_blocks / cand >= 4) {
        cl = cand;
        break;
      }
    cl = debug_knob(B200Q_KNOB_CLUSTER, cl);
    if (cl == 2 || cl == 4) {
      const int per = (pl.k_blocks + cl - 1) / cl;
      if (tiles * cl <= sms && per * (cl - 1) < pl.k_blocks) {
        pl.cluster = cl;
        pl.splits = cl;
        pl.kb_per_split = per;
        pl.partial_bytes = (cl - 1) * bn * kTileA * static_cast<int>(sizeof(float));
      }
    }
  }
  if (pl.splits > 1 && pl.cluster == 1 && tiles * sizeof(unsigned int) > kCounterBytes) return false;
  const int rows16 = swap ? bn : kTileA;
  const int rows8 = swap ? kTileA : bn;
  const int stage_bytes = rows16 * kRow16 + rows8 * kRow8;
  // deeper ring of converted tiles where they are small: the expand -> MMA -> release chain
  // takes about a microsecond per K block, so two buffers cap a narrow tile at 0.5 us per block
  pl.conv_bufs = rows8 <= 64 ? 8 : rows8 <= 128 ? 4 : 2;
  const int fixed = pl.conv_bufs * rows8 * kRow16 + pl.partial_bytes + kStagingBytes + kScaleSmemBytes +
                    kCtrlBytes;
  int stages = (kMaxSmem - fixed) / stage_bytes;
  stages = std::min(stages, kMaxStages);
  stages = std::min(stages, std::max(2, pl.kb_per_split));
  if (stages < 2) return false;
  pl.stages = stages;
  pl.smem_bytes = static_cast<size_t>(stages) * stage_bytes + fixed;
  int cols = 32;
  while (cols < 2 * bn) cols *= 2;
  pl.tmem_cols = cols;
  const long long items = tiles * pl.splits;
  pl.grid = static_cast<int>(std::min<long long>(items, sms));
  pl.ws_bytes = (pl.splits > 1 && pl.cluster == 1)
                    ? kCounterBytes + static_cast<size_t>(tiles) * pl.splits * bn * kTileA * sizeof(float)
                    : 0;
  *plan = pl;
  return true;
}

int launch_w8a16_umma(const GemmArgs& a, const UmmaPlan& plan) {
  if (plan.ws_bytes > 0) {
    if (a.workspace == nullptr || a.workspace_bytes < plan.ws_bytes) return B200Q_ERR_WORKSPACE;
  }
  const int rows16 = plan.swap ? plan.bn : kTileA;
  const int rows8 = plan.swap ? kTileA : plan.bn;
  CUtensorMap tx, tw;
  // activations: [M, 2K bytes], 128-byte boxes; weights: [N, K bytes], 64-byte boxes
  if (!make_tensor_map(a.x, a.M, static_cast<uint64_t>(a.K) * 2, rows16, kRow16, &tx))
    return B200Q_ERR_LAUNCH;
  if (!get_tensor_map(a.w, a.N, a.K, rows8, kRow8, &tw)) return B200Q_ERR_LAUNCH;

  KernelParams kp{};
  kp.rows_a = plan.rows_a;
  kp.rows_b = plan.rows_b;
  kp.bn = plan.bn;
  kp.tiles_a = plan.tiles_a;
  kp.tiles_b = plan.tiles_b;
  kp.k_blocks = plan.k_blocks;
  kp.splits = plan.splits;
  kp.kb_per_split = plan.kb_per_split;
  kp.stages = plan.stages;
  kp.conv_bufs = plan.conv_bufs;
  kp.cluster = plan.cluster;
  kp.partial_bytes = plan.partial_bytes;
  kp.tmem_cols = plan.tmem_cols;
  kp.swap = plan.swap;
  kp.n_channels = a.N;
  kp.is_bf16 = a.dtype == B200Q_DTYPE_BF16 ? 1 : 0;
  kp.w_scales = a.w_scales;
  kp.bias = a.bias;
  kp.out = a.y;
  kp.counters = reinterpret_cast<unsigned int*>(a.workspace);
  kp.partials = plan.ws_bytes > 0
                    ? reinterpret_cast<float*>(static_cast<uint8_t*>(a.workspace) + kCounterBytes)
                    : nullptr;
  kp.status = a.status;
  kp.fast_store = (!plan.swap && (plan.splits == 1 || plan.cluster > 1) && (a.N % 8) == 0 &&
                   (plan.bn % 64) == 0) ? 1 : 0;
  kp.debug_flags = debug_knob(B200Q_KNOB_FLAGS, 0);

  cudaError_t e;
  if (plan.cluster > 1) {
    e = a.dtype == B200Q_DTYPE_BF16 ? launch_kernel<__nv_bfloat16, true>(tx, tw, kp, plan, a.stream)
                                    : launch_kernel<__half, true>(tx, tw, kp, plan, a.stream);
  } else {
    e = a.dtype == B200Q_DTYPE_BF16 ? launch_kernel<__nv_bfloat16, false>(tx, tw, kp, plan, a.stream)
                                    : launch_kernel<__half, false>(tx, tw, kp, plan, a.stream);
  }
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch();
  return B200Q_OK;
}

}  // namespace b200q
