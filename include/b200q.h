/*
 * b200q — C ABI of the B200 (sm_100a) quantized-linear kernels.
 *
 * This header is the drop-in boundary for the quantized linear path of
 * tiny-vLLM (a nano-vllm fork).  Each entry point names the reference interface
 * it stands in for (paths are relative to the reference project root).
 *
 * Conventions shared by every compute entry point
 *   - Plain pointers and sizes only; every pointer is DEVICE memory owned by the
 *     caller.  The library allocates nothing per call and keeps only cached TMA
 *     descriptors and kernel attributes.
 *   - `stream` is a cudaStream_t passed as void*.  Work is always enqueued on
 *     that stream (the reference launches on the legacy default stream instead:
 *     nanovllm/quantization/csrc/w8a8_gemm.cu:438, int8_weight_only_gemm.cu:558),
 *     so calls can be recorded by a CUDA-graph capture of that stream.
 *   - No call synchronises the device and no call falls back to another
 *     implementation: a non-zero return code means nothing was launched.
 *   - Matrices are row-major and dense: x[M,K], qweight[N,K], y[M,N].
 *   - K must be a multiple of 16 (the row pitch of an int8 [rows,K] matrix must
 *     be 16-byte aligned for TMA); all base pointers must be 16-byte aligned.
 *   - Return value: B200Q_OK (0) or one of the B200Q_ERR_* codes below;
 *     b200q_strerror() gives the text.
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200Q_VERSION 2

/* ---- error codes ------------------------------------------------------- */
enum {
  B200Q_OK = 0,
  B200Q_ERR_NULL_POINTER = 1,      /* a required pointer is NULL */
  B200Q_ERR_BAD_SHAPE = 2,         /* M, N or K is <= 0 or overflows int32 indexing */
  B200Q_ERR_UNSUPPORTED_SHAPE = 3, /* K % 16 != 0, or a stride rule is violated */
  B200Q_ERR_MISALIGNED = 4,        /* a pointer is not 16-byte aligned */
  B200Q_ERR_WORKSPACE = 5,         /* workspace is NULL or smaller than b200q_workspace_bytes() */
  B200Q_ERR_UNSUPPORTED_ARCH = 6,  /* current device is not compute capability 10.x */
  B200Q_ERR_LAUNCH = 7,            /* a CUDA runtime/driver call failed (see b200q_last_cuda_error) */
  B200Q_ERR_BAD_ARGUMENT = 8,      /* unknown op / dtype / path id */
  B200Q_ERR_DEVICE_TIMEOUT = 9,    /* a bounded device-side wait gave up (b200q_device_status) */
  B200Q_ERR_SCRATCH_LIMIT = 10     /* problem needs more built-in scratch than B200Q_NOALLOC_SCRATCH_BYTES */
};

/* Size of the scratch area built into the library for b200q_w8a8_gemm_noalloc. */
#define B200Q_NOALLOC_SCRATCH_BYTES (8u << 20)

/* ---- element types of the floating-point side -------------------------- */
enum {
  B200Q_DTYPE_F16 = 0,
  B200Q_DTYPE_BF16 = 1
};

/* ---- operations (for workspace / path queries) ------------------------- */
enum {
  B200Q_OP_ACT_QUANT = 0,
  B200Q_OP_W8A8 = 1,
  B200Q_OP_W8A16 = 2
};

/* ---- kernel families (b200q_select_path ids / b200q_debug_force_path) --- */
enum {
  B200Q_PATH_AUTO = 0,
  B200Q_PATH_SIMT_STREAM = 1, /* weight-streaming SIMT kernel, tiny M                    */
  B200Q_PATH_UMMA = 2,        /* tcgen05 kernel, tokens on the 128-row side (prefill)     */
  B200Q_PATH_UMMA_SWAP = 3,   /* tcgen05 kernel, channels on the 128-row side + split-K   */
  B200Q_PATH_MMA_STREAM = 4   /* weight-streaming mma.sync kernel, in-CTA split-K, M <= 64 */
};

/*
 * Per-token dynamic int8 quantisation of activations:
 *   a_scales[m] = max(max_k |x[m,k]| / 127, 1e-8)            (fp32, IEEE division)
 *   xq[m,k]     = clamp(round_half_even(x[m,k] / a_scales[m]), -127, 127)
 * x is [M,K] with row pitch ldx elements (ldx >= K, ldx % 8 == 0), dtype per
 * x_dtype; xq is dense int8 [M,K]; a_scales is fp32 [M].
 * Replaces nanovllm/quantization/utils.py:28-32 (quantize_int8_per_row_dynamic),
 * called from nanovllm/quantization/w8a8.py:21-23; results are bit-identical to it.
 */
int b200q_act_quant_i8(const void* x, int64_t ldx, int x_dtype, int8_t* xq, float* a_scales,
                       int M, int K, void* stream);

/*
 * The same quantisation fused into the two operations that produce the inputs of the W8A8
 * layers in the reference's model (nanovllm/models/qwen3.py:119-121,160-166), so that the
 * 16-bit activation is never written to and re-read from memory (no counterpart in the
 * reference, which runs the producer and the quantiser as separate steps).
 *
 * b200q_add_rmsnorm_quant_i8 — RMSNorm.forward of nanovllm/layers/layernorm.py:16-50:
 *   s = float(x) + float(residual_in)   (residual_in may be NULL: s = float(x))
 *   residual_out = T(s)                 (skipped when residual_out is NULL; may alias residual_in, not x)
 *   y = T(T(s * rsqrt(mean_k(s^2) + eps)) * weight)
 *   (xq, a_scales) = per-token quantisation of y, bit-identical to b200q_act_quant_i8(y)
 * x, residual_*, y: dense [M, K] of `dtype`; weight: [K] of `dtype`; y is written only when
 * non-NULL.  K % 16 == 0, K <= 16384.
 *
 * b200q_silu_mul_quant_i8 — SiluAndMul.forward of nanovllm/layers/activation.py:11-14:
 *   y = T(silu(float(gate)) * float(up)) with gate = gate_up[:, 0:I], up = gate_up[:, I:2I]
 *   (row pitch ld elements, ld >= 2 I, ld % 8 == 0), then the same quantisation of y.
 * I % 16 == 0, I <= 16384.
 */
int b200q_add_rmsnorm_quant_i8(const void* x, const void* residual_in, const void* weight, float eps,
                               void* residual_out, void* y, int8_t* xq, float* a_scales, int M,
                               int K, int dtype, void* stream);
int b200q_silu_mul_quant_i8(const void* gate_up, int64_t ld, void* y, int8_t* xq, float* a_scales,
                            int M, int I, int dtype, void* stream);

/*
 * W8A8 linear: acc[m,n] = sum_k xq[m,k] * qweight[n,k] (exact int32), then
 *   y[m,n] = out_dtype( (float(acc) * a_scales[m]) * w_scales[n] + bias[n] )
 * bias may be NULL; when given it has dtype out_dtype and length N.
 * Replaces the pybind entry `forward(x_q, a_scales, qweight, w_scales, bias,
 * use_bfloat16)` of nanovllm/quantization/csrc/w8a8_gemm.cpp:16-54 and its
 * launcher w8a8_gemm.cu:426-507 (epilogue arithmetic: w8a8_gemm.cu:387-390).
 * workspace: b200q_workspace_bytes(B200Q_OP_W8A8, M, N, K) bytes (may be 0 -> NULL ok).
 */
int b200q_w8a8_gemm(const int8_t* xq, const float* a_scales, const int8_t* qweight,
                    const float* w_scales, const void* bias, void* y, int M, int N, int K,
                    int out_dtype, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Same contraction as b200q_w8a8_gemm but writes the raw int32 accumulators
 * acc[M,N] and applies no epilogue.  The reference keeps these internal
 * (nanovllm/quantization/csrc/w8a8_gemm.cu:336,377-390; integer MAC loop at
 * w8a8_gemm.cu:165-183); this entry exists so that they can be compared bit for
 * bit with a CPU integer matmul.
 */
int b200q_w8a8_gemm_i32(const int8_t* xq, const int8_t* qweight, int32_t* acc, int M, int N,
                        int K, void* workspace, size_t workspace_bytes, void* stream);

/*
 * W8A16 linear: y[m,n] = x_dtype( scales[n] * sum_k x[m,k] * float(qweight[n,k]) + bias[n] ),
 * fp32 accumulation, x and y and bias share x_dtype (fp16 or bf16).
 * Replaces the pybind entry `forward(x2d, qweight, scales, bias)` of
 * nanovllm/quantization/csrc/int8_weight_only_gemm.cpp:14-43 and its launcher
 * int8_weight_only_gemm.cu:549-618.
 */
int b200q_w8a16_gemm(const void* x, const int8_t* qweight, const float* scales, const void* bias,
                     void* y, int M, int N, int K, int x_dtype, void* workspace,
                     size_t workspace_bytes, void* stream);

/*
 * Scratch bytes the given op needs for the given problem (0 when none).  The
 * first use of a workspace must find it zero-filled; every successful call
 * leaves it zero-filled where that matters, so one zeroed buffer of the maximum
 * size can be shared by all calls that are ordered on one stream.
 */
size_t b200q_workspace_bytes(int op, int M, int N, int K);

/*
 * Name of the kernel family the library would run for this problem, e.g.
 * "umma_i8_128xN" — the counterpart of `select_path(...)` in
 * nanovllm/quantization/csrc/w8a8_gemm.cpp:51-54 and
 * int8_weight_only_gemm.cpp:40-43.  Never NULL.
 */
const char* b200q_select_path(int op, int M, int N, int K);

/* Text for a return code.  Never NULL. */
const char* b200q_strerror(int code);

/* cudaError_t of the most recent failing CUDA call made by this library (0 if none). */
int b200q_last_cuda_error(void);

/*
 * Reads (synchronously, small D2H copy) and clears the device-side status word
 * of the current device.  0 = no kernel gave up a bounded wait since the last
 * read.  Non-zero encodes which wait gave up.  Meant for tests and post-mortems,
 * not for the hot path.
 */
int b200q_device_status(void);

/* Library/ABI version (B200Q_VERSION). */
int b200q_version(void);

/*
 * Test hook: force a kernel family (B200Q_PATH_*) for the GEMM entry points, or
 * B200Q_PATH_AUTO to restore the built-in choice.  A family that cannot run the
 * given problem makes the call return B200Q_ERR_UNSUPPORTED_SHAPE.  Returns the
 * previous setting.  Like every debug knob it applies to the CALLING THREAD only.
 * The reference exposes the same kind of switch through the
 * NANOVLLM_INT8_BACKEND / NANOVLLM_W8A8_BACKEND variables
 * (nanovllm/quantization/cuda.py:46-53).
 */
int b200q_debug_force_path(int path);

/*
 * Test and tuning knobs.  A knob changes which kernel variant runs, how a problem is tiled,
 * or (B200Q_KNOB_FLAGS) switches parts of a kernel off so that their cost can be measured —
 * the last kind makes results WRONG on purpose.  All knobs are unset when the library is
 * loaded, nothing is read from the environment, and a setting is private to the thread
 * that made it: a serving process that never calls b200q_debug_set() cannot be affected.
 * b200q_debug_set returns 0, or -1 for an unknown knob; b200q_debug_reset unsets all knobs
 * of the calling thread.  (The reference's counterparts are environment variables read on
 * every forward: nanovllm/quantization/cuda.py:46-53,249.)
 */
enum {
  B200Q_KNOB_FORCE_PATH = 0,       /* B200Q_PATH_* (same as b200q_debug_force_path) */
  B200Q_KNOB_FLAGS = 1,            /* tcgen05 kernels: 1 skip epilogue arithmetic, 2 skip MMAs, 4 skip output stores */
  B200Q_KNOB_BN = 2,               /* single-CTA kernels: UMMA N */
  B200Q_KNOB_SPLITS = 3,           /* single-CTA kernels: split-K factor */
  B200Q_KNOB_CLUSTER = 4,          /* single-CTA kernels: cluster split-K size */
  B200Q_KNOB_NO_PAIR = 5,          /* 1: never take the CTA-pair kernels */
  B200Q_KNOB_NO_TS = 6,            /* 1: never take the W8A16 kernel with weights in tensor memory */
  B200Q_KNOB_TS_MIN_K = 7,         /* smallest K for that kernel */
  B200Q_KNOB_SIMT_MAX_M = 8,       /* largest M that takes the SIMT cross-check kernels */
  B200Q_KNOB_TILED_ONLY = 9,       /* fused prefill route: 1 = GEMM kernel only, 2 = sum-and-gather only */
  B200Q_KNOB_PAIR_EPILOGUE = 10,   /* CTA-pair kernels: 0 st.global via shared memory, 1 TMA store (default) */
  B200Q_KNOB_W8A16_PAIR_MIN_M = 11,/* smallest M for the expand-once W8A16 route */
  B200Q_KNOB_NO_PDL = 12,          /* 1: plain stream order instead of programmatic dependent launch */
  B200Q_KNOB_WAIT_CYCLES = 13,     /* limit of one wait on a peer GPU, in SM cycles (default about 2e9) */
  B200Q_KNOB_PAIR_MIN_TILES = 14,  /* CTA-pair kernels: fewest 256 x 256 tiles a problem must have */
  B200Q_KNOB_BULK_DECODE = 15,  /* persistent ring-fed decode kernels: 1 never, 2 wherever they can run */
  B200Q_KNOB_BULK_SLOTS = 16,   /* ring depth per consumer warp of those kernels (>= 2; default: what fits) */
  B200Q_KNOB_BULK_WPP = 17,     /* consumer warps per ring of the W8A8 one-token-tile kernel: 1 or 2 (default 2) */
  B200Q_KNOB_COUNT = 20
};
int b200q_debug_set(int knob, int value);
void b200q_debug_reset(void);

/*
 * Reads and clears the device status word like b200q_device_status() (synchronous: call it
 * after the stream has been synchronised) and turns it into a return code: B200Q_OK when no
 * bounded wait gave up since the last read, else B200Q_ERR_DEVICE_TIMEOUT with the word in
 * *status_word (may be NULL).  The reference has no counterpart: its kernels cannot time out,
 * and a failing extension call is turned into a silent fallback
 * (nanovllm/quantization/cuda.py:347-356,493-503); here the failure is reported.
 */
int b200q_check_status(int* status_word);

/* Test hook: number of kernels this library has launched in this process. */
uint64_t b200q_launch_count(void);

/*
 * In-place sum all-reduce of a 16-bit tensor over the tensor-parallel ranks of one node,
 * through peer memory (NVLink).  Replaces `dist.all_reduce(y)` after a row-parallel
 * linear (nanovllm/layers/linear.py:274-275) for tensors that live in a symmetric
 * allocation.  peer_buffers[r] / peer_flag_pads[r] are HOST arrays of `world` DEVICE
 * addresses, as mapped into the calling process: rank r's tensor (same element offset on
 * every rank) and rank r's flag pad (>= 256 bytes, zero-filled once before the first
 * call, never touched by the caller afterwards).  Every rank must make the same sequence
 * of calls; n_elems must be a multiple of 8; world <= 8.  fp32 accumulation in rank
 * order, so all ranks receive bit-identical results.  Waits on peers are bounded (about a
 * second), after which the call's kernel records a status (b200q_device_status) and ends.
 */
int b200q_tp_allreduce(void* const* peer_buffers, void* const* peer_flag_pads, int rank, int world,
                       size_t n_elems, int dtype, void* stream);

/*
 * b200q_tp_allreduce with the data phase done by the NVSwitch (NVLS): multicast_buffer is the
 * MULTICAST address of the symmetric tensor (the mapping through which a store reaches every
 * rank's copy and a reducing load returns the sum of all copies), peer_flag_pads as above.
 * In place; rank r reduces slice r with multimem.ld_reduce (fp32 accumulation in the
 * switch) and broadcasts it with multimem.st.  All ranks receive identical bits; the
 * addition order is the switch's, so the last bit may differ from the rank-ordered sum of
 * b200q_tp_allreduce.  Less link traffic than the two-shot kernel from four ranks up.
 * A wait that runs out sets device status 0x504 / 0x505.
 */
int b200q_tp_allreduce_multimem(void* multicast_buffer, void* const* peer_flag_pads, int rank,
                                int world, size_t n_elems, int dtype, void* stream);

/*
 * Pull variant of b200q_tp_allreduce: every rank reads all ranks' buffers over NVLink and
 * writes the sum (fp32, rank order, bit-identical on all ranks and to b200q_tp_allreduce)
 * into `out`, an ordinary local tensor that must not alias the rank's own input buffer.
 * Nothing is written to a peer, so there is no closing barrier: about a third faster than
 * the two-shot kernel for two ranks, more traffic than it beyond two.  The input buffers
 * must stay untouched until every peer has read them, which the next call of this function
 * or of b200q_tp_allreduce on the same flag pads guarantees (a rank announces itself there
 * only after its own kernel has finished): alternate between two input buffers and keep one
 * such call between two writes to the same buffer.  Same arguments and limits otherwise;
 * a wait that runs out sets device status 0x503.
 */
int b200q_tp_allreduce_pull(void* const* peer_buffers, void* const* peer_flag_pads, void* out,
                            int rank, int world, size_t n_elems, int dtype, void* stream);

/*
 * Row-parallel linear for decode-sized batches with the sum over the tensor-parallel ranks
 * fused into the GEMM kernel: replaces the pair "quantized linear, then dist.all_reduce(y)"
 * of RowParallelLinear.forward (nanovllm/layers/linear.py:265-276) by ONE kernel per rank.
 * Each CTA pushes its partial output tile (rounded to the output type, exactly what
 * b200q_w8a8_gemm / b200q_w8a16_gemm would have stored) into every other rank's receive
 * area with 8-byte peer stores over NVLink (two values and the call number per store, so
 * no fence or separate flag is needed), polls (bounded) its own receive area for the same
 * tile of the peers and stores the fp32 sum, taken in rank order, into y.  The result is
 * bit-identical on every rank and bit-identical to the unfused decode kernel followed by
 * b200q_tp_allreduce.
 *
 * peer_recv / peer_flags are HOST arrays of `world` DEVICE addresses as mapped into the
 * calling process: rank r's receive area (recv_bytes bytes, 256-byte aligned; two halves
 * used alternately, each must hold world * M * N * 4 bytes) and rank r's control words
 * (B200Q_FUSED_FLAG_BYTES).  Both are zero-filled once before the first call and never
 * touched by the caller afterwards.  y is an ordinary local tensor.  Every rank makes the
 * same sequence of calls with the same M, N and dtype (K is the rank's share of the input
 * features), ordered on one stream per rank.
 * Limits: M <= B200Q_FUSED_MAX_M, N % 8 == 0, and the N / 8 CTAs of the kernel must be
 * resident on the device at once; B200Q_ERR_UNSUPPORTED_SHAPE otherwise (nothing is
 * launched and the caller takes the two-kernel route), B200Q_ERR_WORKSPACE when the
 * receive area is too small.  A wait that runs out sets device status 0x601.
 */
#define B200Q_FUSED_MAX_M 64
#define B200Q_FUSED_FLAG_BYTES 256u
int b200q_w8a8_gemm_allreduce(const int8_t* xq, const float* a_scales, const int8_t* qweight,
                              const float* w_scales, const void* bias, void* y, int M, int N,
                              int K, int out_dtype, void* const* peer_recv,
                              void* const* peer_flags, size_t recv_bytes, int rank, int world,
                              void* stream);
int b200q_w8a16_gemm_allreduce(const void* x, const int8_t* qweight, const float* scales,
                               const void* bias, void* y, int M, int N, int K, int x_dtype,
                               void* const* peer_recv, void* const* peer_flags,
                               size_t recv_bytes, int rank, int world, void* stream);

/*
 * Row-parallel W8A8 linear at prefill size with the all-reduce fused in: replaces the pair
 * "quantized linear, then dist.all_reduce(y)" of RowParallelLinear.forward
 * (nanovllm/layers/linear.py:265-276) by two kernels.
 * Rank o owns token rows [o * M / world, (o + 1) * M / world).  Kernel 1 is the CTA-pair
 * tcgen05 GEMM, whose epilogue writes every partial 128 x 256 tile (rounded to the output
 * type, as b200q_w8a8_gemm would store it) straight into the owner's staging area, over
 * NVLink when the owner is a peer: the reduce-scatter half of the all-reduce runs under the
 * GEMM's main loop.  Kernel 2 exchanges one "GEMM complete" flag per peer (bounded wait),
 * adds the `world` partials of the owned rows in rank order in fp32 from local memory and
 * writes the result rows into every rank's output (all-gather half), then waits until
 * every rank has done so.  Results are bit-identical on all ranks and to b200q_w8a8_gemm
 * followed by b200q_tp_allreduce.
 *
 * HOST arrays of `world` DEVICE addresses as mapped into the calling process: peer_y (the
 * output matrix [M, N], same symmetric allocation on every rank), peer_stage (staging area,
 * stage_bytes >= M * N * 2), peer_flags (the control words of the fused kernels above,
 * B200Q_FUSED_FLAG_BYTES; shared call numbering).  Every rank makes the same sequence of
 * calls, ordered on one stream.  Limits: M % (world * 256) == 0, N % 8 == 0;
 * B200Q_ERR_UNSUPPORTED_SHAPE otherwise (nothing launched).  A wait that runs out sets
 * device status 0x701 / 0x702.
 */
int b200q_w8a8_gemm_allreduce_tiled(const int8_t* xq, const float* a_scales, const int8_t* qweight,
                                    const float* w_scales, const void* bias, void* const* peer_y,
                                    int M, int N, int K, int out_dtype, void* const* peer_stage,
                                    size_t stage_bytes, void* const* peer_flags, int rank,
                                    int world, void* stream);

/*
 * Sum all-reduce of a SMALL 16-bit tensor over the tensor-parallel ranks in one NVLink trip
 * (same use as b200q_tp_allreduce, nanovllm/layers/linear.py:274-275, for tensors up to a
 * few hundred kilobytes, where two flag barriers cost more than the data).  x and y are
 * ordinary local tensors of n_elems values (y may be x); every rank pushes x to every peer
 * as 8-byte words tagged with the call number and sums what it receives in rank order
 * (fp32), so all ranks get bit-identical results, equal to those of b200q_tp_allreduce.
 * peer_recv / peer_flags / recv_bytes are the receive areas and control words of the
 * fused kernels above (shared call numbering: calls of the three entry points may be
 * mixed freely as long as every rank makes the same sequence); each half of the receive
 * area must hold world * n_elems * 4 bytes, else B200Q_ERR_WORKSPACE.  n_elems % 8 == 0.
 * A wait that runs out sets device status 0x602.
 */
int b200q_tp_allreduce_small(const void* x, void* y, size_t n_elems, int dtype,
                             void* const* peer_recv, void* const* peer_flags,
                             size_t recv_bytes, int rank, int world, void* stream);

/*
 * The exchange step after a row-parallel linear fused with its consumers: replaces the chain
 *   dist.all_reduce(y)                         (nanovllm/layers/linear.py:274-275)
 *   x, residual = RMSNorm(y, residual)         (nanovllm/layers/layernorm.py:28-40, called at
 *                                               nanovllm/models/qwen3.py:160-166)
 *   x_q, a_scales = quantize_int8_per_row_dynamic(x)   (nanovllm/quantization/w8a8.py:21-23)
 * by ONE kernel per rank.  Rank r owns token rows [r * M / world, (r + 1) * M / world): it
 * sums the partial outputs of all ranks for those rows (fp32, rank order, one rounding to the
 * 16-bit type: the tensor the all-reduce would have produced), adds its shard of the residual
 * stream, writes the new residual shard, applies RMSNorm, quantises, and writes the int8 codes
 * and fp32 scales of its rows into EVERY rank's code / scale buffer, which then hold the whole
 * [M, K] input of the next W8A8 layer.  The residual stream stays sharded by rows: no rank
 * ever needs another rank's rows of it.  Codes, scales and residual are bit-identical to
 * b200q_tp_allreduce followed by b200q_add_rmsnorm_quant_i8 on the owned rows.
 *
 * peer_partials / peer_flag_pads / peer_xq / peer_scales are HOST arrays of `world` DEVICE
 * addresses as mapped into the calling process: rank r's partial output [M, K] (dtype),
 * flag pad (the pads of b200q_tp_allreduce: shared call numbering), code buffer int8 [M, K]
 * and scale buffer fp32 [M] (symmetric allocations).  residual_in (may be NULL) / residual_out
 * (may be NULL, may alias residual_in) / y_local (normalised rows, may be NULL) are LOCAL
 * tensors of M / world rows; weight is [K].  M % world == 0, K % 16 == 0, K <= 16384.  Every
 * rank makes the same sequence of calls.  A wait that runs out sets device status 0x801 /
 * 0x802.  No counterpart in the reference, which runs the three steps one after another.
 */
int b200q_tp_reduce_rmsnorm_quant(void* const* peer_partials, void* const* peer_flag_pads,
                                  const void* residual_in, void* residual_out, const void* weight,
                                  float eps, void* const* peer_xq, void* const* peer_scales,
                                  void* y_local, int M, int K, int rank, int world, int dtype,
                                  void* stream);

/*
 * W8A8 linear for callers that have no way to hand over scratch memory.
 * (No counterpart in the reference: its kernels never need scratch.)
 *
 * Same inputs, outputs and arithmetic as b200q_w8a8_gemm, but without the workspace
 * arguments.  The decode-sized (split-K) kernel needs a few megabytes of scratch for its
 * partial tiles and tile counters; b200q_w8a8_gemm takes that from the caller, who usually
 * gets it from an allocator.  Two kinds of caller cannot do that: an embedder that binds
 * this C ABI directly and owns no device allocator, and a serving process that has already
 * given all remaining HBM to its KV cache after warm-up, where a late cudaMalloc would
 * fail or would have to be carved out of the cache.  For them the scratch lives inside
 * the library, in one fixed device array of B200Q_NOALLOC_SCRATCH_BYTES (8 MiB) that every
 * GPU which loads the library holds until the process exits.
 *
 *  - Nothing is allocated or freed by this call, ever (no cudaMalloc / cudaFree).
 *  - A problem whose split-K scratch would exceed the built-in array is refused with
 *    B200Q_ERR_SCRATCH_LIMIT and nothing is launched; use b200q_w8a8_gemm with a
 *    caller-owned workspace for it.  Problems that need no scratch are never refused.
 *  - The first call on each device looks up the device address of the array (a one-time
 *    host-side query with that device current).  Make that first call during start-up,
 *    before any stream capture is begun.
 *  - All calls share the one array, and the array keeps whatever the last call left in it;
 *    the part that must start at zero (the tile counters) is cleared on the stream at
 *    the start of every call.  Two calls that overlap on the GPU (different streams) race
 *    on the array: keep calls on one device ordered on one stream.
 *  - It always runs the tcgen05 kernel family.  For M <= 64 b200q_w8a8_gemm picks the
 *    weight-streaming kernels instead, which need no scratch at all and are about twice as
 *    fast there (2.5-3.6 us against 6-7.5 us on the Qwen3-0.6B projections): a caller who
 *    can pass workspace = NULL, workspace_bytes = 0 to b200q_w8a8_gemm for those batches
 *    should do that and keep this entry for the larger ones.
 */
int b200q_w8a8_gemm_noalloc(const int8_t* xq, const float* a_scales, const int8_t* qweight,
                            const float* w_scales, const void* bias, void* y, int M, int N,
                            int K, int out_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */
