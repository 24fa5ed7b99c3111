/*
 * C restatement of the integer contraction of the W8A8 path.  TEST INFRASTRUCTURE:
 * used by the tests and by the CPU-baseline leg of the benchmark only.
 *
 * acc[m][n] = sum_k (int)x_q[m][k] * (int)qweight[n][k], exact in int32 — the
 * multiply-accumulate loop of nanovllm/quantization/csrc/w8a8_gemm.cu:165-183.
 * Parity status: pinned through tests/golden/quant_linear_golden.npz (field
 * acc_i32, produced by the reference's own Python functions with unit scales in
 * float64, which is exact for these magnitudes).
 *
 * Built by oracle/build_oracle.py:  gcc -O3 -fopenmp -shared -fPIC
 */
#include <stdint.h>

#if defined(__GNUC__) && defined(__x86_64__)
#define CLONES __attribute__((target_clones("arch=skylake-avx512", "avx2", "default")))
#else
#define CLONES
#endif

CLONES static int32_t dot_i8(const int8_t* a, const int8_t* b, int k) {
  int32_t s = 0;
  for (int i = 0; i < k; ++i) s += (int32_t)a[i] * (int32_t)b[i];
  return s;
}

void w8a8_int32_gemm(const int8_t* x_q, const int8_t* qweight, int32_t* acc, int M, int N, int K) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    const int8_t* xr = x_q + (int64_t)m * K;
    for (int n = 0; n < N; ++n) acc[(int64_t)m * N + n] = dot_i8(xr, qweight + (int64_t)n * K, K);
  }
}
