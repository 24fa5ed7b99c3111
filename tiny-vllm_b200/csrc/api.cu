// C ABI of libb200q: argument validation, kernel-family choice, launches.
// Nothing here allocates device memory, synchronises, or falls back to a CPU path.
#include <cuda_runtime.h>

#include <atomic>
#include <climits>
#include <cstdint>

#include "common.h"

namespace b200q {

// Device-side status word: a kernel whose bounded wait gave up writes a non-zero code here.
__device__ int g_device_status = 0;

namespace {
std::atomic<int> g_last_cuda_error{0};
std::atomic<uint64_t> g_launches{0};

// Debug knobs of the calling thread (common.h): value and "is set" per knob.
struct Knobs {
  int value[B200Q_KNOB_COUNT];
  bool set[B200Q_KNOB_COUNT];
};
thread_local Knobs t_knobs{};

constexpr int kMaxDevices = 64;

struct DeviceInfo {
  std::atomic<int> ready{0};
  int cc_major = 0;
  int sms = 0;
  int* status_ptr = nullptr;
};
DeviceInfo g_dev[kMaxDevices];

DeviceInfo* device_info() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  DeviceInfo& d = g_dev[dev];
  if (d.ready.load(std::memory_order_acquire) == 0) {
    int major = 0, sms = 0;
    cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    void* p = nullptr;
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&p, g_device_status);
    if (e != cudaSuccess) {
      note_cuda_error(e);
      return nullptr;
    }
    d.cc_major = major;
    d.sms = sms;
    d.status_ptr = static_cast<int*>(p);
    d.ready.store(1, std::memory_order_release);
  }
  return &d;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_dims(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return B200Q_ERR_BAD_SHAPE;
  if (static_cast<long long>(M) * N > INT_MAX || static_cast<long long>(M) * K > INT_MAX ||
      static_cast<long long>(N) * K > INT_MAX)
    return B200Q_ERR_BAD_SHAPE;
  if ((K % 16) != 0) return B200Q_ERR_UNSUPPORTED_SHAPE;
  return B200Q_OK;
}

// Kernel family for a W8A8 problem when nothing is forced.
// The weight-streaming mma.sync kernel re-reads the activations once per 8 output channels,
// so its range shrinks as N grows; thresholds from graph-replayed launches of the
// Qwen3-0.6B projections at M = 32, 48, 64 (e.g. M = 48: 4.6 vs 7.6 us for 2048 -> 1024,
// 7.3 vs 6.4 us for 1024 -> 6144).
// Matrices of 8 MB and more (the 8B model): the ring-fed persistent kernels take M <= 32
// (M <= 16 for the widest projections: 24576 channels at M = 32 run 29.9 us there against
// 24.1 us on the tcgen05 kernel), the tcgen05 kernels the rest; the register-streaming kernel's
// activation re-reads, N / 8 x M x K bytes from L2, rule it out (M = 64: 35-101 us against 13-24).
int auto_path_w8a8(int M, int N, int K) {
  if (M <= debug_knob(B200Q_KNOB_SIMT_MAX_M, 0)) return B200Q_PATH_SIMT_STREAM;
  if (static_cast<long long>(N) * K >= (8ll << 20))
    return (M <= 16 || (M <= 32 && N < 16384)) ? B200Q_PATH_MMA_STREAM : B200Q_PATH_UMMA;
  if (M <= 32 || (M <= 48 && N <= 4096) || (M <= 64 && N <= 2048)) return B200Q_PATH_MMA_STREAM;
  return B200Q_PATH_UMMA;
}

// Kernel family for a W8A16 problem when nothing is forced.
// Same for W8A16, where the tcgen05 kernel's expansion stage costs more at small M
// (M = 64: 7.2 vs 17.7 us for 2048 -> 1024, 12.4 vs 11.0 us for 1024 -> 6144).
// Matrices of 8 MB and more: the ring-fed kernel takes one token tile (M <= 16); beyond it the
// register-streaming kernel re-reads N / 8 x M x 2 K bytes of activations from L2 (M = 32 on
// 24576 x 4096: 79 us against 52 us for the tcgen05 kernel at M = 64).
int auto_path_w8a16(int M, int N, int K) {
  if (M <= debug_knob(B200Q_KNOB_SIMT_MAX_M, 0)) return B200Q_PATH_SIMT_STREAM;
  if (static_cast<long long>(N) * K >= (8ll << 20))
    return M <= 16 ? B200Q_PATH_MMA_STREAM : B200Q_PATH_UMMA;
  if (M <= 48 || (M <= 64 && N <= 4096)) return B200Q_PATH_MMA_STREAM;
  return B200Q_PATH_UMMA;
}

int resolve_path(int op, int M, int N, int K) {
  const int forced = debug_knob(B200Q_KNOB_FORCE_PATH, B200Q_PATH_AUTO);
  if (forced != B200Q_PATH_AUTO) return forced;
  return op == B200Q_OP_W8A16 ? auto_path_w8a16(M, N, K) : auto_path_w8a8(M, N, K);
}

int run_w8a8(GemmArgs& a) {
  DeviceInfo* d = device_info();
  if (d == nullptr) return B200Q_ERR_LAUNCH;
  if (d->cc_major != 10) return B200Q_ERR_UNSUPPORTED_ARCH;
  a.status = d->status_ptr;
  const int path = resolve_path(B200Q_OP_W8A8, a.M, a.N, a.K);
  if (path == B200Q_PATH_SIMT_STREAM) {
    cudaError_t e = launch_w8a8_simt(a);
    if (e != cudaSuccess) {
      note_cuda_error(e);
      return B200Q_ERR_LAUNCH;
    }
    return B200Q_OK;
  }
  if (path == B200Q_PATH_MMA_STREAM) {
    if (!mma_decode_applicable(a.M)) return B200Q_ERR_UNSUPPORTED_SHAPE;
    cudaError_t e = bulk_decode_applicable(a.M, a.N, a.K, false) ? launch_w8a8_bulk_decode(a)
                                                          : launch_w8a8_mma_decode(a);
    if (e != cudaSuccess) {
      note_cuda_error(e);
      return B200Q_ERR_LAUNCH;
    }
    return B200Q_OK;
  }
  if (path == B200Q_PATH_UMMA && umma_pair_applicable(a.M, a.N, a.K, a.acc_out != nullptr))
    return launch_w8a8_umma_pair(a);
  if (path == B200Q_PATH_UMMA || path == B200Q_PATH_UMMA_SWAP) {
    UmmaPlan plan;
    if (!umma_make_plan(B200Q_OP_W8A8, a.M, a.N, a.K, path == B200Q_PATH_UMMA_SWAP, &plan))
      return B200Q_ERR_UNSUPPORTED_SHAPE;
    return launch_w8a8_umma(a, plan);
  }
  return B200Q_ERR_BAD_ARGUMENT;
}

}  // namespace

bool pdl_enabled() { return debug_knob(B200Q_KNOB_NO_PDL, 0) == 0; }

int debug_knob(int knob, int dflt) {
  if (knob < 0 || knob >= B200Q_KNOB_COUNT) return dflt;
  return t_knobs.set[knob] ? t_knobs.value[knob] : dflt;
}

int sm_count() {
  DeviceInfo* d = device_info();
  return d != nullptr && d->sms > 0 ? d->sms : 148;
}

int device_cc_major() {
  DeviceInfo* d = device_info();
  return d != nullptr ? d->cc_major : 0;
}

int* device_status_ptr() {
  DeviceInfo* d = device_info();
  return d != nullptr ? d->status_ptr : nullptr;
}

void note_cuda_error(cudaError_t e) { g_last_cuda_error.store(static_cast<int>(e)); }
void count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n)); }

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_act_quant_i8(const void* x, int64_t ldx, int x_dtype, int8_t* xq, float* a_scales, int M,
                       int K, void* stream) {
  if (x == nullptr || xq == nullptr || a_scales == nullptr) return B200Q_ERR_NULL_POINTER;
  if (M <= 0 || K <= 0 || static_cast<long long>(M) * K > INT_MAX) return B200Q_ERR_BAD_SHAPE;
  if (x_dtype != B200Q_DTYPE_F16 && x_dtype != B200Q_DTYPE_BF16) return B200Q_ERR_BAD_ARGUMENT;
  if ((K % 16) != 0 || ldx < K || (ldx % 8) != 0) return B200Q_ERR_UNSUPPORTED_SHAPE;
  if (!aligned16(x) || !aligned16(xq) || (reinterpret_cast<uintptr_t>(a_scales) & 3u) != 0)
    return B200Q_ERR_MISALIGNED;
  DeviceInfo* d = device_info();
  if (d == nullptr) return B200Q_ERR_LAUNCH;
  if (d->cc_major != 10) return B200Q_ERR_UNSUPPORTED_ARCH;
  cudaError_t e =
      launch_act_quant(x, ldx, x_dtype, xq, a_scales, M, K, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return B200Q_ERR_LAUNCH;
  }
  return B200Q_OK;
}

int b200q_w8a8_gemm(const int8_t* xq, const float* a_scales, const int8_t* qweight,
                    const float* w_scales, const void* bias, void* y, int M, int N, int K,
                    int out_dtype, void* workspace, size_t workspace_bytes, void* stream) {
  if (xq == nullptr || a_scales == nullptr || qweight == nullptr || w_scales == nullptr ||
      y == nullptr)
    return B200Q_ERR_NULL_POINTER;
  if (int rc = check_dims(M, N, K)) return rc;
  if (out_dtype != B200Q_DTYPE_F16 && out_dtype != B200Q_DTYPE_BF16) return B200Q_ERR_BAD_ARGUMENT;
  if (!aligned16(xq) || !aligned16(qweight) || !aligned16(y) || !aligned16(w_scales) ||
      (reinterpret_cast<uintptr_t>(a_scales) & 3u) != 0 ||
      (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 1u) != 0) ||
      (workspace != nullptr && !aligned16(workspace)))
    return B200Q_ERR_MISALIGNED;
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
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  return run_w8a8(a);
}

int b200q_w8a8_gemm_allreduce(const int8_t* xq, const float* a_scales, const int8_t* qweight,
                              const float* w_scales, const void* bias, void* y, int M, int N,
                              int K, int out_dtype, void* const* peer_recv,
                              void* const* peer_flags, size_t recv_bytes, int rank, int world,
                              void* stream) {
  if (xq == nullptr || a_scales == nullptr || qweight == nullptr || w_scales == nullptr ||
      y == nullptr)
    return B200Q_ERR_NULL_POINTER;
  if (int rc = check_dims(M, N, K)) return rc;
  if (out_dtype != B200Q_DTYPE_F16 && out_dtype != B200Q_DTYPE_BF16) return B200Q_ERR_BAD_ARGUMENT;
  if (!aligned16(xq) || !aligned16(qweight) || !aligned16(y) ||
      (reinterpret_cast<uintptr_t>(a_scales) & 3u) != 0 ||
      (reinterpret_cast<uintptr_t>(w_scales) & 3u) != 0 ||
      (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 1u) != 0))
    return B200Q_ERR_MISALIGNED;
  DeviceInfo* d = device_info();
  if (d == nullptr) return B200Q_ERR_LAUNCH;
  if (d->cc_major != 10) return B200Q_ERR_UNSUPPORTED_ARCH;
  GemmArgs a{};
  a.x = xq;
  a.w = qweight;
  a.a_scales = a_scales;
  a.w_scales = w_scales;
  a.bias = bias;
  a.y = y;
  a.M = M;
  a.N = N;
  a.K = K;
  a.dtype = out_dtype;
  a.status = d->status_ptr;
  a.stream = static_cast<cudaStream_t>(stream);
  return launch_w8a8_mma_decode_fused(a, peer_recv, peer_flags, recv_bytes, rank, world);
}

int b200q_w8a8_gemm_allreduce_tiled(const int8_t* xq, const float* a_scales, const int8_t* qweight,
                                    const float* w_scales, const void* bias, void* const* peer_y,
                                    int M, int N, int K, int out_dtype, void* const* peer_stage,
                                    size_t stage_bytes, void* const* peer_flags, int rank,
                                    int world, void* stream) {
  if (xq == nullptr || a_scales == nullptr || qweight == nullptr || w_scales == nullptr ||
      peer_y == nullptr || peer_stage == nullptr || peer_flags == nullptr)
    return B200Q_ERR_NULL_POINTER;
  if (int rc = check_dims(M, N, K)) return rc;
  if (out_dtype != B200Q_DTYPE_F16 && out_dtype != B200Q_DTYPE_BF16) return B200Q_ERR_BAD_ARGUMENT;
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return B200Q_ERR_BAD_ARGUMENT;
  if ((N % 8) != 0 || (M % (world * 256)) != 0) return B200Q_ERR_UNSUPPORTED_SHAPE;
  if (!aligned16(xq) || !aligned16(qweight) ||
      (reinterpret_cast<uintptr_t>(a_scales) & 3u) != 0 ||
      (reinterpret_cast<uintptr_t>(w_scales) & 3u) != 0 ||
      (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 1u) != 0))
    return B200Q_ERR_MISALIGNED;
  if (static_cast<size_t>(M) * N * 2 > stage_bytes) return B200Q_ERR_WORKSPACE;
  for (int r = 0; r < world; ++r) {
    if (peer_y[r] == nullptr || peer_stage[r] == nullptr || peer_flags[r] == nullptr)
      return B200Q_ERR_NULL_POINTER;
    if (!aligned16(peer_y[r]) || !aligned16(peer_stage[r])) return B200Q_ERR_MISALIGNED;
  }
  DeviceInfo* d = device_info();
  if (d == nullptr) return B200Q_ERR_LAUNCH;
  if (d->cc_major != 10) return B200Q_ERR_UNSUPPORTED_ARCH;
  GemmArgs a{};
  a.x = xq;
  a.w = qweight;
  a.a_scales = a_scales;
  a.w_scales = w_scales;
  a.bias = bias;
  a.M = M;
  a.N = N;
  a.K = K;
  a.dtype = out_dtype;
  a.status = d->status_ptr;
  a.stream = static_cast<cudaStream_t>(stream);
  // test hook: 1 = GEMM kernel only, 2 = sum-and-gather kernel only (two calls make one)
  const int only = debug_knob(B200Q_KNOB_TILED_ONLY, 0);
  if (!(only & 2)) {
    if (int rc = launch_w8a8_umma_pair_scatter(a, peer_stage, rank, world)) return rc;
  }
  if (only & 1) return B200Q_OK;
  return launch_tp_reduce_gather(peer_stage[rank], peer_y, peer_flags, rank, world, M, N,
                                 out_dtype, a.stream);
}

int b200q_w8a16_gemm_allreduce(const void* x, const int8_t* qweight, const float* scales,
                               const void* bias, void* y, int M, int N, int K, int x_dtype,
                               void* const* peer_recv, void* const* peer_flags,
                               size_t recv_bytes, int rank, int world, void* stream) {
  if (x == nullptr || qweight == nullptr || scales == nullptr || y == nullptr)
    return B200Q_ERR_NULL_POINTER;
  if (int rc = check_dims(M, N, K)) return rc;
  if (x_dtype != B200Q_DTYPE_F16 && x_dtype != B200Q_DTYPE_BF16) return B200Q_ERR_BAD_ARGUMENT;
  if (!aligned16(x) || !aligned16(qweight) || !aligned16(y) ||
      (reinterpret_cast<uintptr_t>(scales) & 3u) != 0 ||
      (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 1u) != 0))
    return B200Q_ERR_MISALIGNED;
  DeviceInfo* d = device_info();
  if (d == nullptr) return B200Q_ERR_LAUNCH;
  if (d->cc_major != 10) return B200Q_ERR_UNSUPPORTED_ARCH;
  GemmArgs a{};
  a.x = x;
  a.w = qweight;
  a.w_scales = scales;
  a.bias = bias;
  a.y = y;
  a.M = M;
  a.N = N;
  a.K = K;
  a.dtype = x_dtype;
  a.status = d->status_ptr;
  a.stream = static_cast<cudaStream_t>(stream);
  return launch_w8a16_mma_decode_fused(a, peer_recv, peer_flags, recv_bytes, rank, world);
}

int b200q_w8a8_gemm_i32(const int8_t* xq, const int8_t* qweight, int32_t* acc, int M, int N, int K,
                        void* workspace, size_t workspace_bytes, void* stream) {
  if (xq == nullptr || qweight == nullptr || acc == nullptr) return B200Q_ERR_NULL_POINTER;
  if (int rc = check_dims(M, N, K)) return rc;
  if (!aligned16(xq) || !aligned16(qweight) || !aligned16(acc) ||
      (workspace != nullptr && !aligned16(workspace)))
    return B200Q_ERR_MISALIGNED;
  GemmArgs a{};
  a.x = xq;
  a.w = qweight;
  a.acc_out = acc;
  a.M = M;
  a.N = N;
  a.K = K;
  a.dtype = B200Q_DTYPE_BF16;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  return run_w8a8(a);
}

int b200q_w8a16_gemm(const void* x, const int8_t* qweight, const float* scales, const void* bias,
                     void* y, int M, int N, int K, int x_dtype, void* workspace,
                     size_t workspace_bytes, void* stream) {
  if (x == nullptr || qweight == nullptr || scales == nullptr || y == nullptr)
    return B200Q_ERR_NULL_POINTER;
  if (int rc = check_dims(M, N, K)) return rc;
  if (x_dtype != B200Q_DTYPE_F16 && x_dtype != B200Q_DTYPE_BF16) return B200Q_ERR_BAD_ARGUMENT;
  if (!aligned16(x) || !aligned16(qweight) || !aligned16(y) || !aligned16(scales) ||
      (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 1u) != 0) ||
      (workspace != nullptr && !aligned16(workspace)))
    return B200Q_ERR_MISALIGNED;
  DeviceInfo* d = device_info();
  if (d == nullptr) return B200Q_ERR_LAUNCH;
  if (d->cc_major != 10) return B200Q_ERR_UNSUPPORTED_ARCH;
  GemmArgs a{};
  a.x = x;
  a.w = qweight;
  a.w_scales = scales;
  a.bias = bias;
  a.y = y;
  a.M = M;
  a.N = N;
  a.K = K;
  a.dtype = x_dtype;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.status = d->status_ptr;
  a.stream = static_cast<cudaStream_t>(stream);
  const int path = resolve_path(B200Q_OP_W8A16, M, N, K);
  if (path == B200Q_PATH_SIMT_STREAM) {
    cudaError_t e = launch_w8a16_simt(a);
    if (e != cudaSuccess) {
      note_cuda_error(e);
      return B200Q_ERR_LAUNCH;
    }
    return B200Q_OK;
  }
  if (path == B200Q_PATH_MMA_STREAM) {
    if (!mma_decode_applicable(M)) return B200Q_ERR_UNSUPPORTED_SHAPE;
    cudaError_t e = bulk_decode_applicable(M, N, K, true) ? launch_w8a16_bulk_decode(a)
                                                    : launch_w8a16_mma_decode(a);
    if (e != cudaSuccess) {
      note_cuda_error(e);
      return B200Q_ERR_LAUNCH;
    }
    return B200Q_OK;
  }
  if (path == B200Q_PATH_UMMA && umma16_pair_applicable(M, N, K)) return launch_w8a16_umma_pair(a);
  if (path == B200Q_PATH_UMMA && umma16_ts_applicable(M, N, K)) return launch_w8a16_umma_ts(a);
  if (path == B200Q_PATH_UMMA || path == B200Q_PATH_UMMA_SWAP) {
    UmmaPlan plan;
    if (!umma16_make_plan(M, N, K, path == B200Q_PATH_UMMA_SWAP, &plan))
      return B200Q_ERR_UNSUPPORTED_SHAPE;
    return launch_w8a16_umma(a, plan);
  }
  return B200Q_ERR_BAD_ARGUMENT;
}

size_t b200q_workspace_bytes(int op, int M, int N, int K) {
  if (op == B200Q_OP_W8A16 && check_dims(M, N, K) == B200Q_OK &&
      resolve_path(op, M, N, K) == B200Q_PATH_UMMA) {
    if (umma16_pair_applicable(M, N, K)) return umma16_pair_workspace_bytes(N, K);
    if (umma16_ts_applicable(M, N, K)) return 0;
  }
  if (op != B200Q_OP_W8A8 && op != B200Q_OP_W8A16) return 0;
  if (check_dims(M, N, K) != B200Q_OK) return 0;
  const int path = resolve_path(op, M, N, K);
  if (path != B200Q_PATH_UMMA && path != B200Q_PATH_UMMA_SWAP) return 0;
  UmmaPlan plan;
  const bool ok = op == B200Q_OP_W8A8
                      ? umma_make_plan(op, M, N, K, path == B200Q_PATH_UMMA_SWAP, &plan)
                      : umma16_make_plan(M, N, K, path == B200Q_PATH_UMMA_SWAP, &plan);
  return ok ? plan.ws_bytes : 0;
}

const char* b200q_select_path(int op, int M, int N, int K) {
  if (op == B200Q_OP_ACT_QUANT) return K <= 1024 ? "act_quant_warp_per_row" : "act_quant_multiwarp_row";
  if (op != B200Q_OP_W8A8 && op != B200Q_OP_W8A16) return "invalid_op";
  if (check_dims(M, N, K) != B200Q_OK) return "unsupported_shape";
  const int path = resolve_path(op, M, N, K);
  const bool a16 = op == B200Q_OP_W8A16;
  switch (path) {
    case B200Q_PATH_SIMT_STREAM:
      return a16 ? "simt_stream_w8a16" : "simt_stream_dp4a";
    case B200Q_PATH_MMA_STREAM:
      if (bulk_decode_applicable(M, N, K, a16))
        return a16 ? "bulk_ring_w8a16_persistent" : "bulk_ring_s8_persistent";
      return a16 ? "mma_stream_w8a16_splitk" : "mma_stream_s8_splitk";
    case B200Q_PATH_UMMA:
      if (!a16 && umma_pair_applicable(M, N, K, false)) return "umma_i8_pair_tokens256";
      if (a16 && umma16_pair_applicable(M, N, K)) return "umma_f16_pair_expand_once_tokens256";
      if (a16 && umma16_ts_applicable(M, N, K)) return "umma_f16_tmem_weights_channels256";
      return a16 ? "umma_f16_expand_tokens128" : "umma_i8_tokens128";
    case B200Q_PATH_UMMA_SWAP:
      return a16 ? "umma_f16_expand_channels128_splitk" : "umma_i8_channels128_splitk";
    default:
      return "invalid_path";
  }
}

const char* b200q_strerror(int code) {
  switch (code) {
    case B200Q_OK:
      return "ok";
    case B200Q_ERR_NULL_POINTER:
      return "a required pointer is NULL";
    case B200Q_ERR_BAD_SHAPE:
      return "M, N or K is not positive or too large";
    case B200Q_ERR_UNSUPPORTED_SHAPE:
      return "unsupported shape (K must be a multiple of 16; row pitch rules)";
    case B200Q_ERR_MISALIGNED:
      return "a pointer is not sufficiently aligned (16 bytes)";
    case B200Q_ERR_WORKSPACE:
      return "workspace missing or smaller than b200q_workspace_bytes()";
    case B200Q_ERR_UNSUPPORTED_ARCH:
      return "device is not compute capability 10.x (B200)";
    case B200Q_ERR_LAUNCH:
      return "a CUDA call failed (see b200q_last_cuda_error)";
    case B200Q_ERR_BAD_ARGUMENT:
      return "unknown op, dtype or path id";
    case B200Q_ERR_DEVICE_TIMEOUT:
      return "a bounded device-side wait gave up";
    case B200Q_ERR_SCRATCH_LIMIT:
      return "problem needs more scratch than the library's built-in 8 MiB array; "
             "use b200q_w8a8_gemm with a caller-owned workspace";
    default:
      return "unknown error code";
  }
}

int b200q_last_cuda_error(void) { return g_last_cuda_error.load(); }

int b200q_device_status(void) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int));
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return -1;
  }
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
  }
  return v;
}

int b200q_check_status(int* status_word) {
  const int v = b200q_device_status();
  if (status_word != nullptr) *status_word = v;
  if (v < 0) return B200Q_ERR_LAUNCH;
  return v == 0 ? B200Q_OK : B200Q_ERR_DEVICE_TIMEOUT;
}

int b200q_version(void) { return B200Q_VERSION; }

int b200q_debug_force_path(int path) {
  if (path < B200Q_PATH_AUTO || path > B200Q_PATH_MMA_STREAM) return -1;
  const int prev = debug_knob(B200Q_KNOB_FORCE_PATH, B200Q_PATH_AUTO);
  t_knobs.value[B200Q_KNOB_FORCE_PATH] = path;
  t_knobs.set[B200Q_KNOB_FORCE_PATH] = path != B200Q_PATH_AUTO;
  return prev;
}

int b200q_debug_set(int knob, int value) {
  if (knob < 0 || knob >= B200Q_KNOB_COUNT) return -1;
  t_knobs.value[knob] = value;
  t_knobs.set[knob] = true;
  return 0;
}

void b200q_debug_reset(void) { t_knobs = Knobs{}; }

uint64_t b200q_launch_count(void) { return g_launches.load(); }

}  // extern "C"
