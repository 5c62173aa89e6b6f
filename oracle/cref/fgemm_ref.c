/* TEST INFRASTRUCTURE — plain-C restatement of the loop nests the reference emits for cpu_gemm.
 * Nothing in the product links this file.
 *
 * The reference's emitter (specializations/cpu_gemm/emit_c.py:83-155) prints the loop nest it is
 * given with `double` buffers and a fixed row stride of 1000 (emit_c.py:29-44), which aliases rows
 * once a dimension reaches 1000.  These functions are the same nests with the true leading
 * dimensions, so they stay valid at any size:
 *   oracle_dgemm_naive / oracle_sgemm_naive   the untuned nest of make_matmul_stmt
 *       (Search/interface.py:66-116): for i0<M: for i1<N: for i2<K: C[i0,i1] += A[i0,i2]*B[i2,i1]
 *   oracle_dgemm_tuned / oracle_sgemm_tuned   the nest after the schedule the reference's README
 *       quotes (README.md:47,71-75): tile i0 32, tile i1 32, reorder i1_inner i2, vectorize i1_inner,
 *       parallel i0_outer — i.e. omp parallel for over i0_outer, omp simd over i1_inner.
 * C must be zeroed by the caller (the runner memsets it, runner.py:180).  M and N must be multiples
 * of 32 for the tuned forms, as the tile tactic demands (VeriTac/Tactic/Tile.lean:296).
 */
#include <stddef.h>

#define NAIVE(NAME, T)                                                                          \
  void NAME(const T *A, const T *B, T *C, long M, long N, long K) {                             \
    for (long i0 = 0; i0 < M; i0++)                                                             \
      for (long i1 = 0; i1 < N; i1++)                                                           \
        for (long i2 = 0; i2 < K; i2++) C[i0 * N + i1] = C[i0 * N + i1] + A[i0 * K + i2] * B[i2 * N + i1]; \
  }

#define TUNED(NAME, T)                                                                          \
  void NAME(const T *A, const T *B, T *C, long M, long N, long K) {                             \
    _Pragma("omp parallel for") for (long i0_outer = 0; i0_outer < M / 32; i0_outer++)          \
      for (long i0_inner = 0; i0_inner < 32; i0_inner++)                                        \
        for (long i1_outer = 0; i1_outer < N / 32; i1_outer++)                                  \
          for (long i2 = 0; i2 < K; i2++) {                                                     \
            _Pragma("omp simd") for (long i1_inner = 0; i1_inner < 32; i1_inner++)              \
              C[(i0_outer * 32 + i0_inner) * N + (i1_outer * 32 + i1_inner)] =                  \
                  C[(i0_outer * 32 + i0_inner) * N + (i1_outer * 32 + i1_inner)] +              \
                  A[(i0_outer * 32 + i0_inner) * K + i2] * B[i2 * N + (i1_outer * 32 + i1_inner)]; \
          }                                                                                     \
  }

NAIVE(oracle_dgemm_naive, double)
NAIVE(oracle_sgemm_naive, float)
TUNED(oracle_dgemm_tuned, double)
TUNED(oracle_sgemm_tuned, float)
