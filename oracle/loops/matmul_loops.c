/*
 * CPU restatement, in plain C, of what the reference executes for an f32
 * linalg.matmul when no optimising stage is given: lh-run always appends
 * `convert-linalg-to-loops` and `llvm-lowering.yaml` (lighthouse/lh_run.py:106-107),
 * which turn the op into the loop nest
 *     for i, for j, for k:  C[i,j] = C[i,j] + A[i,k] * B[k,j]
 * with every operation in f32 and k ascending. TEST INFRASTRUCTURE: used as the
 * parity checker and as the timed CPU baseline, never by the product path.
 *
 * lh_oracle_matmul_loops      the literal nest (i, j, k), rows split over threads
 * lh_oracle_matmul_loops_ikj  same sums in the same k order per element, loops
 *                             interchanged to (i, k, j) so the compiler vectorises
 *                             over j; bit-identical results, much faster — this is
 *                             the baseline that is timed at full size
 * lh_oracle_matmul_bias_relu  bf16-rounded inputs given as f32: f32 accumulate,
 *                             + bias, ReLU (emit_mlp_layer,
 *                             lighthouse/ingress/mlir_gen/gpu_mlp_payload.py:110-156)
 */
#include <stddef.h>
#include <stdint.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int lh_oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void lh_oracle_matmul_loops(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      float acc = C[i * N + j];
      for (int64_t k = 0; k < K; ++k) acc = acc + A[i * K + k] * B[k * N + j];
      C[i * N + j] = acc;
    }
}

void lh_oracle_matmul_loops_ikj(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M; ++i)
    for (int64_t k = 0; k < K; ++k) {
      const float a = A[i * K + k];
      float* c = C + i * N;
      const float* b = B + k * N;
      for (int64_t j = 0; j < N; ++j) c[j] = c[j] + a * b[j];
    }
}

void lh_oracle_matmul_bias_relu(const float* A, const float* B, const float* bias, float* D, int64_t M,
                                int64_t N, int64_t K, int relu) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M; ++i) {
    float* d = D + i * N;
    for (int64_t j = 0; j < N; ++j) d[j] = 0.0f;
    for (int64_t k = 0; k < K; ++k) {
      const float a = A[i * K + k];
      const float* b = B + k * N;
      for (int64_t j = 0; j < N; ++j) d[j] = d[j] + a * b[j];
    }
    for (int64_t j = 0; j < N; ++j) {
      float v = d[j] + (bias ? bias[j] : 0.0f);
      if (relu && v < 0.0f) v = 0.0f;
      d[j] = v;
    }
  }
}
