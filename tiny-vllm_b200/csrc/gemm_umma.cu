// W8A8 GEMM on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
// One persistent, warp-specialised kernel:
//   warp 0      TMA producer: streams 128-byte-wide K blocks of both operands into a
//               shared-memory ring (128-byte swizzle), one mbarrier per stage.
//   warp 1      UMMA issuer: tcgen05.mma kind::i8 (int8 x int8 -> int32), accumulators
//               in TMEM, double-buffered so that the epilogue of tile i overlaps the
//               main loop of tile i+1.
//   warps 2-5   epilogue: tcgen05.ld -> (acc * a_scale) * w_scale + bias -> f16/bf16
//               -> global, or raw int32, or split-K partials + last-arriver reduction.
//
// The operand on the 128-row side of the UMMA tile ("A side") is the activation
// matrix for prefill-shaped problems and the weight matrix for decode-shaped ones
// ("swap"), where the few tokens become the N extent of the instruction and K is
// split over CTAs so that the whole GPU streams the weights.
//
// Arithmetic follows nanovllm/quantization/csrc/w8a8_gemm.cu:165-183 (exact int32
// accumulation) and :387-390 (float(acc) * a_scale * w_scale + bias, cast).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "common.h"
#include "ptx_sm100.cuh"
#include "w8a8_device.cuh"

namespace b200q {
namespace {

// CLUSTER: K split over a cluster of p.cluster CTAs, reduced in the leader's shared memory.
template <typename OutT, int MODE, bool CLUSTER>
__global__ void __launch_bounds__(kThreads, 1)
w8a8_umma_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b, const KernelParams p) {
  // Swizzled operand tiles need 1024-byte alignment; the dynamic shared window starts on
  // such a boundary (checked below, the kernel refuses to run otherwise).
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t stage_bytes = kTileA * kBlockK + p.bn * kBlockK;
  int32_t* partial = reinterpret_cast<int32_t*>(smem + static_cast<size_t>(p.stages) * stage_bytes);
  uint8_t* staging = reinterpret_cast<uint8_t*>(partial) + p.partial_bytes;
  float* s_ws = reinterpret_cast<float*>(staging + kStagingBytes);
  uint8_t* ctrl = reinterpret_cast<uint8_t*>(s_ws) + kScaleSmemBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* tfull_bar = empty_bar + kMaxStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* pfull_bar = tempty_bar + 2;  // cluster leader: partial tiles have arrived
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pfull_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [2]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = ptx::smem_u32(smem);
  if ((smem_base & 1023u) != 0u) {  // uniform over the CTA: nothing has been set up yet
    if (threadIdx.x == 0) atomicCAS(p.status, 0, 0x200);
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(full_bar + s), 1);
      ptx::mbar_init(ptx::smem_u32(empty_bar + s), 1);
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
    ptx::tma_prefetch_desc(&tmap_a);
    ptx::tma_prefetch_desc(&tmap_b);
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
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(empty_bar + stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t bar = ptx::smem_u32(full_bar + stage);
          const uint32_t sa = smem_base + stage * stage_bytes;
          const uint32_t sb = sa + kTileA * kBlockK;
          ptx::mbar_arrive_expect_tx(bar, stage_bytes);
          ptx::tma_load_2d(sa, &tmap_a, bar, kb * kBlockK, tile_a * kTileA);
          ptx::tma_load_2d(sb, &tmap_b, bar, kb * kBlockK, tile_b * p.bn);
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
      const uint32_t idesc = ptx::umma_idesc(2u, 1u, kTileA, static_cast<uint32_t>(p.bn));
      int stage = 0;
      uint32_t phase = 0;
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
          if (!ptx::mbar_wait(ptx::smem_u32(full_bar + stage), phase, abort_flag)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * stage_bytes;
          const uint32_t sb = sa + kTileA * kBlockK;
          const uint64_t a_desc = ptx::umma_desc_k_sw128(sa);
          const uint64_t b_desc = ptx::umma_desc_k_sw128(sb);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            if (p.debug_flags & 2) break;
            // advancing K by 32 bytes inside the swizzled row = +2 in 16-byte units
            ptx::umma_i8_ss(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc,
                            (kb > kb0 || k > 0) ? 1u : 0u);
          }
          ptx::umma_commit(ptx::smem_u32(empty_bar + stage));
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) ptx::umma_commit(ptx::smem_u32(tfull_bar + buf));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    // Warp (2 + e) owns TMEM lanes [32*(warp & 3), +32) and the 64-column groups
    // e/4, e/4 + 2, ... of the tile.
    const int epi_warp = warp - 2;
    const int quarter = warp & 3;
    const int half = epi_warp >> 2;
    const int row_in_tile = quarter * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    const int n_chunks_tile = p.bn >> 5;                 // 32-column chunks in the tile
    const int n_groups_tile = (n_chunks_tile + 1) >> 1;  // 64-column groups (last may be half)
    const int my_groups = (n_groups_tile - half + 1) >> 1;
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
      float a_s = 0.f;
      float* ws_tile = s_ws + buf * 256;
      if (clustered && split > 0) {
        // K split over the cluster: hand this CTA's partial tile (exact int32 sums) to the
        // leader (cluster rank 0 = split 0) through its shared memory, [split - 1][column][row]
        if (!ptx::mbar_wait(ptx::smem_u32(tfull_bar + buf), tphase, abort_flag)) break;
        ptx::tc_fence_after_sync();
        const uint32_t taddr_p = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                 static_cast<uint32_t>(buf * p.bn);
        const uint32_t dst0 = ptx::map_to_cta(ptx::smem_u32(partial), 0) +
                              (static_cast<uint32_t>((split - 1) * p.bn) * kTileA + row_in_tile) * 4u;
        for (int c = half * 2; c < n_chunks_tile; c += 4) {   // this warp's 64-column groups
          for (int h = 0; h < 2 && c + h < n_chunks_tile; ++h) {
            uint32_t v[32];
            ptx::tmem_ld_32x32b_x32(taddr_p + (c + h) * 32, v);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              ptx::st_shared_cluster_u32(dst0 + static_cast<uint32_t>((c + h) * 32 + j) * (kTileA * 4u),
                                         v[j]);
          }
        }
        ptx::tc_fence_before_sync();
        ptx::mbar_arrive(ptx::smem_u32(tempty_bar + buf));
        ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(pfull_bar), 0));  // release: stores first
        continue;
      }
      if (fast && !(p.debug_flags & 8)) {
        // channel scales of this tile -> shared memory (while the main loop still runs)
        const int col = tile_b * p.bn + epi_tid;
        if (epi_tid < p.bn) ws_tile[epi_tid] = col < p.rows_b ? __ldg(p.w_scales + col) : 0.f;
        const int row = tile_a * kTileA + row_in_tile;
        if (row < p.rows_a) a_s = __ldg(p.a_scales + row);
        ptx::named_bar_sync(2, kEpiThreads);
      }
      if (!ptx::mbar_wait(ptx::smem_u32(tfull_bar + buf), tphase, abort_flag)) break;
      if (clustered && !ptx::mbar_wait_cluster(ptx::smem_u32(pfull_bar), 0u, abort_flag)) break;
      ptx::tc_fence_after_sync();
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buf * p.bn);
      // leader of a cluster: add the peers' partial tiles (int32: exact in any order)
      auto add_partials = [&](int c0, uint32_t (&v)[32]) {
        for (int sp = 1; sp < p.cluster; ++sp) {
          const int32_t* src = partial + static_cast<size_t>((sp - 1) * p.bn + c0) * kTileA + row_in_tile;
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += static_cast<uint32_t>(src[j * kTileA]);
        }
      };
      int32_t* mine = nullptr;
      if (p.splits > 1 && !clustered)
        mine = p.partials + (static_cast<size_t>(t) * p.splits + split) * p.bn * kTileA + row_in_tile;

      // One 32-column chunk in registers -> its destination (generic paths).
      auto consume = [&](int c0, const uint32_t (&v)[32]) {
        if (p.splits > 1 && !clustered) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            __stcg(mine + static_cast<size_t>(c0 + j) * kTileA, static_cast<int32_t>(v[j]));
        } else {
          emit_chunk<OutT, MODE>(p, tile_a, tile_b, row_in_tile, c0, v);
        }
      };

      // Each group = two 32-column TMEM reads issued together.  The reads of group g+1 are
      // issued as soon as the registers of group g have been converted, so they are in
      // flight while group g is written out.
      uint32_t va[32], vb[32];
      if (p.debug_flags & 16) {
#pragma unroll
        for (int j = 0; j < 32; ++j) va[j] = vb[j] = j + lane;
      }
      auto issue = [&](int g) {
        const int c = (half + 2 * g) * 2;  // first 32-column chunk of the group
        if (p.debug_flags & 16) return;
        ptx::tmem_ld_32x32b_x32(taddr + c * 32, va);
        if (c + 1 < n_chunks_tile) ptx::tmem_ld_32x32b_x32(taddr + (c + 1) * 32, vb);
      };
      if (my_groups > 0) issue(0);
      for (int g = 0; g < my_groups; ++g) {
        const int c = (half + 2 * g) * 2;
        const bool two = c + 1 < n_chunks_tile;
        ptx::tmem_ld_wait();
        if (p.debug_flags & 1) {
          if (g + 1 < my_groups) issue(g + 1);
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
            convert_chunk<OutT, true>(p, ws_tile + c * 32, a_s, col0, lane, 0, slab, va);
            if (two) convert_chunk<OutT, true>(p, ws_tile + c * 32 + 32, a_s, col0 + 32, lane, 1, slab, vb);
          } else {
            convert_chunk<OutT, false>(p, ws_tile + c * 32, a_s, col0, lane, 0, slab, va);
            if (two) convert_chunk<OutT, false>(p, ws_tile + c * 32 + 32, a_s, col0 + 32, lane, 1, slab, vb);
          }
          if (g + 1 < my_groups) issue(g + 1);
          __syncwarp();
          if (!(p.debug_flags & 4)) store_group<OutT>(p, slab, lane, row0, col0);
          __syncwarp();
        } else {
          consume(c * 32, va);
          if (two) consume(c * 32 + 32, vb);
          if (g + 1 < my_groups) issue(g + 1);
        }
      }
      // all TMEM reads of this thread are complete: hand the accumulator back
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(ptx::smem_u32(tempty_bar + buf));

      if (p.splits > 1 && !clustered) {
        // split-K: the last CTA to arrive for this tile sums all partial tiles.
        __threadfence();
        ptx::named_bar_sync(1, kEpiThreads);
        if (epi_tid == 0) {
          const unsigned int old = atomicAdd(p.counters + t, 1u);
          const int last = (old == static_cast<unsigned int>(p.splits - 1));
          if (last) p.counters[t] = 0u;  // every split has arrived: leave the counter clean
          last_flag[it & 1] = last;
        }
        ptx::named_bar_sync(1, kEpiThreads);
        if (last_flag[it & 1]) {
          __threadfence();
          const int32_t* base =
              p.partials + static_cast<size_t>(t) * p.splits * p.bn * kTileA + row_in_tile;
          for (int ch = half; ch < n_chunks_tile; ch += 2) {
            const int c0 = ch * 32;
            uint32_t v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
            for (int s = 0; s < p.splits; ++s) {
              const int32_t* src = base + static_cast<size_t>(s) * p.bn * kTileA;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                v[j] += static_cast<uint32_t>(__ldcg(src + static_cast<size_t>(c0 + j) * kTileA));
            }
            emit_chunk<OutT, MODE>(p, tile_a, tile_b, row_in_tile, c0, v);
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
    atomicCAS(p.status, 0, 0x100 | (static_cast<int>(blockIdx.x) << 12));
  }
}

// ------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(sym);
    else note_cuda_error(e == cudaSuccess ? cudaErrorUnknown : e);
  });
  return fn;
}

struct MapKey {
  const void* base;
  uint64_t rows, row_bytes;
  uint32_t box_rows, box_bytes;
  int device;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && row_bytes == o.row_bytes &&
           box_rows == o.box_rows && box_bytes == o.box_bytes && device == o.device;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h ^= k.rows * 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.row_bytes * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    h ^= (static_cast<size_t>(k.box_rows) << 8) ^ static_cast<size_t>(k.device) ^
         (static_cast<size_t>(k.box_bytes) << 20);
    return h;
  }
};

}  // namespace

bool make_tensor_map(const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                     uint32_t box_bytes, CUtensorMap* out) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    note_cuda_error(cudaErrorInvalidValue);
    return false;
  }
  return true;
}

// Cached variant for matrices that keep their address (weights): encoding costs about a
// microsecond of host time.
bool get_tensor_map(const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                    uint32_t box_bytes, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  int dev = 0;
  cudaGetDevice(&dev);
  MapKey key{base, rows, row_bytes, box_rows, box_bytes, dev};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  CUtensorMap m;
  if (!make_tensor_map(base, rows, row_bytes, box_rows, box_bytes, &m)) return false;
  {
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, m);
  }
  *out = m;
  return true;
}

namespace {

int round_up(int v, int m) { return (v + m - 1) / m * m; }

template <typename OutT, int MODE, bool CLUSTER>
cudaError_t launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const KernelParams& kp,
                           const UmmaPlan& plan, cudaStream_t stream) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = w8a8_umma_kernel<OutT, MODE, CLUSTER>;
  if (dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  return launch_clustered(plan.cluster, true, kern, plan.grid, kThreads, plan.smem_bytes, stream, ta,
                          tb, kp);
}

template <typename OutT, int MODE>
cudaError_t launch_kernel(const CUtensorMap& ta, const CUtensorMap& tb, const KernelParams& kp,
                          const UmmaPlan& plan, cudaStream_t stream) {
  return plan.cluster > 1 ? launch_variant<OutT, MODE, true>(ta, tb, kp, plan, stream)
                          : launch_variant<OutT, MODE, false>(ta, tb, kp, plan, stream);
}

}  // namespace

bool umma_make_plan(int op, int M, int N, int K, int swap, UmmaPlan* plan) {
  if (op != B200Q_OP_W8A8) return false;
  if (M <= 0 || N <= 0 || K <= 0 || (K % 16) != 0) return false;
  UmmaPlan pl{};
  pl.swap = swap;
  pl.rows_a = swap ? N : M;
  pl.rows_b = swap ? M : N;
  const int sms = sm_count();
  pl.k_blocks = (K + kBlockK - 1) / kBlockK;
  int bn = pl.rows_b >= 256 ? 256 : round_up(pl.rows_b, 32);
  if (!swap && pl.rows_b >= 256) {
    // Prefer the N tile that leaves the fewest idle SMs in the last wave.
    const int ta = (pl.rows_a + kTileA - 1) / kTileA;
    double best = 1e30;
    for (int cand : {256, 128, 64}) {
      const int tiles = ta * ((pl.rows_b + cand - 1) / cand);
      const int waves = (tiles + sms - 1) / sms;
      // cost model: a wave costs its MMA time (proportional to cand) plus a fixed part
      const double cost = waves * (cand + 48.0);
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
  if (tiles * 2 <= sms && pl.k_blocks >= 64) {
    splits = static_cast<int>(sms / tiles);
    splits = std::min(splits, pl.k_blocks / 32);
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
  if (op == B200Q_OP_W8A8 && !swap && pl.splits == 1) {
    // worth it when the leader's K loop gets at least 8 blocks (about 1.7 us) shorter: the
    // cluster launch, its two barriers and the reduction cost about a microsecond
    int cl = 1;
    for (int cand : {4, 2})
      if (tiles * cand <= sms && pl.k_blocks / cand >= 3 &&
          pl.k_blocks - (pl.k_blocks + cand - 1) / cand >= 8) {
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
        pl.partial_bytes = (cl - 1) * bn * kTileA * static_cast<int>(sizeof(int32_t));
      }
    }
  }
  if (pl.splits > 1 && pl.cluster == 1 && tiles * sizeof(unsigned int) > kCounterBytes) return false;
  const int stage_bytes = kTileA * kBlockK + bn * kBlockK;
  const int kFixedSmem = pl.partial_bytes + kStagingBytes + kScaleSmemBytes + kCtrlBytes;
  int stages = (kMaxSmem - kFixedSmem) / stage_bytes;
  stages = std::min(stages, kMaxStages);
  stages = std::min(stages, std::max(2, pl.kb_per_split * 2));
  pl.stages = stages;
  pl.smem_bytes = static_cast<size_t>(stages) * stage_bytes + kFixedSmem;
  int cols = 32;
  while (cols < 2 * bn) cols *= 2;
  pl.tmem_cols = cols;
  const long long items = tiles * pl.splits;
  pl.grid = static_cast<int>(std::min<long long>(items, sms));
  pl.ws_bytes = (pl.splits > 1 && pl.cluster == 1)
                    ? kCounterBytes + static_cast<size_t>(tiles) * pl.splits * bn * kTileA * sizeof(int32_t)
                    : 0;
  *plan = pl;
  return true;
}

int launch_w8a8_umma(const GemmArgs& a, const UmmaPlan& plan) {
  if (plan.ws_bytes > 0) {
    if (a.workspace == nullptr || a.workspace_bytes < plan.ws_bytes) return B200Q_ERR_WORKSPACE;
  }
  const void* base_a = plan.swap ? static_cast<const void*>(a.w) : a.x;
  const void* base_b = plan.swap ? a.x : static_cast<const void*>(a.w);
  CUtensorMap ta, tb;
  // the weight map is cached (fixed address), the activation map is encoded per call
  const auto map_a = plan.swap ? get_tensor_map : make_tensor_map;
  const auto map_b = plan.swap ? make_tensor_map : get_tensor_map;
  if (!map_a(base_a, plan.rows_a, a.K, kTileA, kBlockK, &ta)) return B200Q_ERR_LAUNCH;
  if (!map_b(base_b, plan.rows_b, a.K, plan.bn, kBlockK, &tb)) return B200Q_ERR_LAUNCH;
  // Prefill orientation, 16-bit output, no split-K: outputs are transposed through shared
  // memory so that every store instruction writes complete 128-byte lines.
  const bool fast_store = !plan.swap && a.acc_out == nullptr &&
                          (plan.splits == 1 || plan.cluster > 1) && (a.N % 8) == 0 &&
                          (plan.bn % 64) == 0;

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
  kp.cluster = plan.cluster;
  kp.partial_bytes = plan.partial_bytes;
  kp.tmem_cols = plan.tmem_cols;
  kp.swap = plan.swap;
  kp.n_channels = a.N;
  kp.n_tokens = a.M;
  kp.a_scales = a.a_scales;
  kp.w_scales = a.w_scales;
  kp.bias = a.bias;
  kp.out = a.acc_out != nullptr ? static_cast<void*>(a.acc_out) : a.y;
  kp.counters = reinterpret_cast<unsigned int*>(a.workspace);
  kp.partials = plan.ws_bytes > 0
                    ? reinterpret_cast<int32_t*>(static_cast<uint8_t*>(a.workspace) + kCounterBytes)
                    : nullptr;
  kp.status = a.status;
  kp.fast_store = fast_store ? 1 : 0;
  kp.debug_flags = debug_knob(B200Q_KNOB_FLAGS, 0);

  cudaError_t e;
  if (a.acc_out != nullptr) {
    e = launch_kernel<__nv_bfloat16, OUT_I32>(ta, tb, kp, plan, a.stream);
  } else if (a.dtype == B200Q_DTYPE_BF16) {
    e = launch_kernel<__nv_bfloat16, OUT_SCALED>(ta, tb, kp, plan, a.stream);
  } else {
    e = launch_kernel<__half, OUT_SCALED>(ta, tb, kp, plan, a.stream);
  }
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  count_launch();
  return B200Q_OK;
}

// ------------------------------------------------------------ built-in scratch variant
// Scratch for b200q_w8a8_gemm_noalloc: tile counters first, split-K partial tiles after
// them.  Lives in every GPU context that loads the library, for the life of the process.
static __device__ __align__(256) unsigned char g_noalloc_scratch[B200Q_NOALLOC_SCRATCH_BYTES];

namespace {

// Device address of g_noalloc_scratch on the current device.  In host code the array's
// name is only a handle for the runtime, not an address a kernel could use, so the real
// address is asked for once per device (with that device current) and remembered.
unsigned char* noalloc_scratch_ptr() {
  static std::mutex mu;
  static unsigned char* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> g(mu);
  if (cached[dev] == nullptr) {
    unsigned char* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      note_cuda_error(e == cudaSuccess ? cudaErrorUnknown : e);
      return nullptr;
    }
    cached[dev] = ptr;
  }
  return cached[dev];
}

}  // namespace

}  // namespace b200q

extern "C" int b200q_w8a8_gemm_noalloc(const int8_t* xq, const float* a_scales,
                                       const int8_t* qweight, const float* w_scales,
                                       const void* bias, void* y, int M, int N, int K,
                                       int out_dtype, void* stream) {
  using namespace b200q;
  // Cheap argument checks first: same rules as b200q_w8a8_gemm.
  if (xq == nullptr || a_scales == nullptr || qweight == nullptr || w_scales == nullptr ||
      y == nullptr)
    return B200Q_ERR_NULL_POINTER;
  if (M <= 0 || N <= 0 || K <= 0 || static_cast<long long>(M) * N > 0x7FFFFFFFLL ||
      static_cast<long long>(M) * K > 0x7FFFFFFFLL || static_cast<long long>(N) * K > 0x7FFFFFFFLL)
    return B200Q_ERR_BAD_SHAPE;
  if ((K % 16) != 0) return B200Q_ERR_UNSUPPORTED_SHAPE;
  if (out_dtype != B200Q_DTYPE_F16 && out_dtype != B200Q_DTYPE_BF16) return B200Q_ERR_BAD_ARGUMENT;
  auto misaligned = [](const void* p, uintptr_t mask) {
    return (reinterpret_cast<uintptr_t>(p) & mask) != 0;
  };
  if (misaligned(xq, 15) || misaligned(qweight, 15) || misaligned(y, 15) ||
      misaligned(w_scales, 15) || misaligned(a_scales, 3) || (bias != nullptr && misaligned(bias, 1)))
    return B200Q_ERR_MISALIGNED;
  const int cc = device_cc_major();
  if (cc == 0) return B200Q_ERR_LAUNCH;
  if (cc != 10) return B200Q_ERR_UNSUPPORTED_ARCH;

  // Decode-sized token counts take the split-K kernel (channels on the 128-row side),
  // larger ones the prefill orientation, which needs no scratch for most shapes.
  UmmaPlan plan;
  if (!umma_make_plan(B200Q_OP_W8A8, M, N, K, M <= 256 ? 1 : 0, &plan))
    return B200Q_ERR_UNSUPPORTED_SHAPE;
  if (plan.ws_bytes > B200Q_NOALLOC_SCRATCH_BYTES) return B200Q_ERR_SCRATCH_LIMIT;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned char* scratch = nullptr;
  if (plan.ws_bytes > 0) {
    scratch = noalloc_scratch_ptr();  // first call on a device: one-time address look-up
    if (scratch == nullptr) return B200Q_ERR_LAUNCH;
    // The array still holds the previous call's data.  Only the tile counters have to
    // start at zero; the partial tiles are fully overwritten before they are read.
    const size_t counter_bytes =
        static_cast<size_t>(plan.tiles_a) * plan.tiles_b * sizeof(unsigned int);
    cudaError_t e = cudaMemsetAsync(scratch, 0, counter_bytes, st);
    if (e != cudaSuccess) {
      note_cuda_error(e);
      return B200Q_ERR_LAUNCH;
    }
  }
  GemmArgs a{};
  a.x = xq;
  a.w = qweight;
  a.a_scales = a_scales;
  a.w_scales = w_scales;
  a.bias = bias;
  a.y = y;
  a.acc_out = nullptr;
  a.M = M;
  a.N = N;
  a.K = K;
  a.dtype = out_dtype;
  a.workspace = scratch;
  a.workspace_bytes = plan.ws_bytes > 0 ? B200Q_NOALLOC_SCRATCH_BYTES : 0;
  a.status = device_status_ptr();
  a.stream = st;
  if (a.status == nullptr) return B200Q_ERR_LAUNCH;
  return launch_w8a8_umma(a, plan);
}
