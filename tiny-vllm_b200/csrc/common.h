// Internal declarations shared by the translation units of libb200q.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/b200q.h"

namespace b200q {

// One linear-layer problem, in the vocabulary of the layer: M tokens, K input
// features, N output channels.
struct GemmArgs {
  const void* x;          // int8 [M,K] (W8A8) or f16/bf16 [M,K] (W8A16)
  const int8_t* w;        // int8 [N,K]
  const float* a_scales;  // fp32 [M]  (W8A8 only)
  const float* w_scales;  // fp32 [N]
  const void* bias;       // [N] in `dtype`, or nullptr
  void* y;                // [M,N] in `dtype`            (nullptr in int32 mode)
  int32_t* acc_out;       // [M,N] raw accumulators      (int32 mode only)
  int M, N, K;
  int dtype;              // B200Q_DTYPE_*
  void* workspace;
  size_t workspace_bytes;
  int* status;            // device status word of the current device
  cudaStream_t stream;
};

// Tiling of one problem onto the tcgen05 kernel.  "A side" is the operand that
// fills the 128 rows of the UMMA tile, "B side" the one that fills its columns.
struct UmmaPlan {
  int swap;          // 0: A = tokens, B = channels; 1: A = channels, B = tokens
  int rows_a, rows_b;
  int bn;            // B-side tile (UMMA N), multiple of 32, <= 256
  int tiles_a, tiles_b;
  int k_blocks;      // ceil(K_bytes / 128)
  int splits;        // split-K factor
  int kb_per_split;
  int stages;        // shared-memory ring depth
  int conv_bufs;     // W8A16 only: ring depth of the converted (16-bit) weight tiles
  int cluster;       // CTAs per cluster that split K and reduce through shared memory (1 = off)
  int partial_bytes; // shared memory for the partial tiles the cluster leader receives
  int tmem_cols;     // power of two >= 2 * bn
  int grid;          // CTAs launched (persistent)
  size_t smem_bytes;
  size_t ws_bytes;   // counters + split-K partials (0 when splits == 1)
};

constexpr size_t kCounterBytes = 16384;  // zero-initialised tile counters at workspace start

// Number of SMs of the current device (cached).
int sm_count();
// Compute-capability major of the current device (0 on error) and the device address of
// its status word (nullptr on error); both cached per device.
int device_cc_major();
int* device_status_ptr();

// act_quant.cu
cudaError_t launch_act_quant(const void* x, int64_t ldx, int x_dtype, int8_t* xq, float* a_scales,
                             int M, int K, cudaStream_t stream);

// gemm_simt.cu
cudaError_t launch_w8a8_simt(const GemmArgs& a);
cudaError_t launch_w8a16_simt(const GemmArgs& a);

// gemm_mma_decode.cu: weight-streaming mma.sync kernels for M <= 64
bool mma_decode_applicable(int M);
cudaError_t launch_w8a8_mma_decode(const GemmArgs& a);
cudaError_t launch_w8a16_mma_decode(const GemmArgs& a);
// The same kernels with the row-parallel sum over peer memory fused in; return B200Q_* codes.
int launch_w8a8_mma_decode_fused(const GemmArgs& a, void* const* peer_recv,
                                 void* const* peer_flags, size_t recv_bytes, int rank, int world);
int launch_w8a16_mma_decode_fused(const GemmArgs& a, void* const* peer_recv,
                                  void* const* peer_flags, size_t recv_bytes, int rank, int world);

// gemm_bulk_decode.cu: persistent decode kernels for large matrices; a producer warp streams
// weights and activations through a shared-memory ring of bulk asynchronous copies
bool bulk_decode_applicable(int M, int N, int K, bool a16);
cudaError_t launch_w8a8_bulk_decode(const GemmArgs& a);
cudaError_t launch_w8a16_bulk_decode(const GemmArgs& a);

// gemm_umma.cu
bool umma_make_plan(int op, int M, int N, int K, int swap, UmmaPlan* plan);
// Returns a B200Q_* code.
int launch_w8a8_umma(const GemmArgs& a, const UmmaPlan& plan);

// gemm_umma.cu: TMA descriptor of a dense row-major matrix viewed as bytes [rows, row_bytes],
// box = box_bytes (128: 128-byte swizzle, 64: 64-byte swizzle) x box_rows, zero fill outside.
// make_tensor_map encodes on every call (activations and outputs: their addresses change from
// call to call); get_tensor_map keeps the result in a per-process cache (weights: same
// address for the life of the model).
bool make_tensor_map(const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                     uint32_t box_bytes, CUtensorMap* out);
bool get_tensor_map(const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                    uint32_t box_bytes, CUtensorMap* out);

// Test and tuning hooks (B200Q_KNOB_* of b200q.h).  Every knob is unset (the built-in
// behaviour) until the CALLING THREAD sets it through b200q_debug_set(); nothing is read from
// the environment, so a stray variable can never change what a kernel computes.
int debug_knob(int knob, int dflt);
// Limit of one wait on a peer GPU in SM cycles: about a second unless a test shortened it.
inline long long peer_wait_limit_cycles() {
  const int k = debug_knob(B200Q_KNOB_WAIT_CYCLES, 0);
  return k > 0 ? static_cast<long long>(k) : 2000000000LL;
}

// gemm_umma_pair.cu: CTA-pair (cta_group::2) variant for prefill-sized W8A8 problems
bool umma_pair_applicable(int M, int N, int K, bool raw_int32_out);
int launch_w8a8_umma_pair(const GemmArgs& a);
// Row-parallel prefill: the pair kernel writing its partial tiles to the owners' staging areas
// (reduce-scatter under the main loop), and the kernel that sums and gathers them.
int launch_w8a8_umma_pair_scatter(const GemmArgs& a, void* const* peer_stage, int rank,
                                  int world);
int launch_tp_reduce_gather(const void* stage, void* const* peer_y,
                            void* const* peer_ctl, int rank, int world, int M, int N, int dtype,
                            cudaStream_t stream);

// gemm_umma_pair.cu: W8A16 prefill route — weights expanded once per call into the
// workspace, then the 16-bit CTA-pair kernel
bool umma16_pair_applicable(int M, int N, int K);
size_t umma16_pair_workspace_bytes(int N, int K);
int launch_w8a16_umma_pair(const GemmArgs& a);

// gemm_umma_w8a16.cu
bool umma16_make_plan(int M, int N, int K, int swap, UmmaPlan* plan);
int launch_w8a16_umma(const GemmArgs& a, const UmmaPlan& plan);

// gemm_umma_w8a16_ts.cu: prefill variant with the expanded weights in tensor memory
bool umma16_ts_applicable(int M, int N, int K);
int launch_w8a16_umma_ts(const GemmArgs& a);

// Launches `kernel` so that it may overlap its start-up (barrier set-up, TMEM allocation,
// descriptor prefetch, launch latency) with the tail of the previous kernel in the stream
// (programmatic dependent launch).  Only for kernels that call ptx::grid_dependency_wait()
// before their first access to global memory.  B200Q_KNOB_NO_PDL turns the overlap off.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
cudaError_t launch_clustered(int cluster, bool overlap, void (*kernel)(KArgs...), dim3 grid,
                             dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = (overlap && pdl_enabled()) ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cluster > 1) {  // grid.x must be a multiple of the cluster size
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = static_cast<unsigned int>(cluster);
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
cudaError_t launch_maybe_overlapped(bool overlap, void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                    size_t smem, cudaStream_t stream, Args&&... args) {
  return launch_clustered(1, overlap, kernel, grid, block, smem, stream,
                          static_cast<Args&&>(args)...);
}
template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args&&... args) {
  return launch_maybe_overlapped(true, kernel, grid, block, smem, stream,
                                 static_cast<Args&&>(args)...);
}

void note_cuda_error(cudaError_t e);
void count_launch(int n = 1);

}  // namespace b200q
