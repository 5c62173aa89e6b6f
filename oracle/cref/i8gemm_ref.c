/* TEST INFRASTRUCTURE — plain-C restatement of the reference's int8 GEMM arithmetic.
 * Nothing in the product links this file; tests and the CPU-baseline legs of the benchmark do.
 *
 * oracle_i8_scalar_ref   the reference's exact scalar loop, veritac_scalar_ref in the C it emits
 *                        (specializations/gemmini_gemm/backend.py:711-720; Python twin :569-580):
 *                        s += (int32)A[i*K+t] * (int32)B[t*N+j] in increasing t.
 * oracle_i8_tiled_ref    the same sum in the order the baseline schedule visits it
 *                        (gen_baseline, backend.py:278-302): i,j,k blocks of 16, the first K block
 *                        overwrites the 16x16 accumulator tile, later ones accumulate, then the tile
 *                        is moved out (compute semantics backend.py:490-529).  OpenMP over row
 *                        blocks; this is the timed CPU baseline.
 * oracle_i8_lcg_inputs   deterministic_inputs(mode="lcg") (backend.py:583-602).
 */
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

void oracle_i8_scalar_ref(const int8_t *A, const int8_t *B, int32_t *C, long M, long N, long K) {
  for (long i = 0; i < M; ++i)
    for (long j = 0; j < N; ++j) {
      int32_t s = 0;
      for (long t = 0; t < K; ++t) s += (int32_t)A[i * K + t] * (int32_t)B[t * N + j];
      C[i * N + j] = s;
    }
}

/* rows [row0, row1) of C only, so a bounded sample of a large product can be timed. */
void oracle_i8_tiled_ref(const int8_t *A, const int8_t *B, int32_t *C, long M, long N, long K, long row0,
                         long row1) {
  const long it0 = row0 / 16, it1 = row1 / 16, jt = N / 16, kt = K / 16;
  (void)M;
#pragma omp parallel for schedule(static)
  for (long i = it0; i < it1; ++i) {
    for (long j = 0; j < jt; ++j) {
      int32_t acc[16][16];
      for (long kk = 0; kk < kt; ++kk) {
        const int8_t *Ad = A + (i * K + kk) * 16; /* tile (i,kk), row stride K */
        const int8_t *Bd = B + (kk * N + j) * 16; /* tile (kk,j), row stride N */
        for (int r = 0; r < 16; ++r)
          for (int c = 0; c < 16; ++c) {
            int32_t s = 0;
            for (int t = 0; t < 16; ++t) s += (int32_t)Ad[r * K + t] * (int32_t)Bd[t * N + c];
            acc[r][c] = (kk == 0) ? s : acc[r][c] + s;
          }
      }
      int32_t *Cd = C + (i * N + j) * 16;
      for (int r = 0; r < 16; ++r) memcpy(Cd + r * N, acc[r], 16 * sizeof(int32_t));
    }
  }
}

void oracle_i8_lcg_inputs(int8_t *A, long na, int8_t *B, long nb, uint32_t seed) {
  uint32_t x = seed;
  for (long i = 0; i < na; ++i) {
    x = 1103515245u * x + 12345u;
    A[i] = (int8_t)((int)((x >> 16) % 256u) - 128);
  }
  for (long i = 0; i < nb; ++i) {
    x = 1103515245u * x + 12345u;
    B[i] = (int8_t)((int)((x >> 16) % 256u) - 128);
  }
}

/* torchrun exports OMP_NUM_THREADS=1; the timed baseline asks for the cores it is allowed instead. */
void oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
