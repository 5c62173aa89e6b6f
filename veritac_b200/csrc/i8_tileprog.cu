// Executes the arithmetic content of a validated Gemmini command stream that is not a plain GEMM:
// every output tile is a sum of 16x16x16 int8 products, exactly what a sequence of
// preload/compute/mvout commands leaves in the accumulator rows that get moved out
// (reference specializations/gemmini_gemm/backend.py:490-553; step semantics
// VeriTac/Gemmini/Engine.lean:38-82).  One CTA of 256 threads per output tile, one output cell
// per thread; the two operand tiles of each term are staged in shared memory.  Streams handled
// here are the small ones the reference itself caps at a few thousand commands, so the kernel is
// written for clarity, not throughput.
#include "runtime.h"

namespace vt {
namespace {

__global__ void __launch_bounds__(256)
i8_tile_program_kernel(const int8_t* __restrict__ A, const int8_t* __restrict__ B, int32_t* __restrict__ C,
                       int64_t lda, int64_t ldb, int64_t ldc, const int64_t* __restrict__ c_off,
                       const int64_t* __restrict__ term_begin, const int64_t* __restrict__ a_off,
                       const int64_t* __restrict__ b_off) {
  __shared__ int a_s[16][17];
  __shared__ int b_s[16][17];
  const int64_t t = blockIdx.x;
  const int r = threadIdx.x >> 4, c = threadIdx.x & 15;
  int32_t acc = 0;
  const int64_t j0 = term_begin[t], j1 = term_begin[t + 1];
  for (int64_t j = j0; j < j1; ++j) {
    a_s[r][c] = A[a_off[j] + r * lda + c];
    b_s[r][c] = B[b_off[j] + r * ldb + c];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) acc += a_s[r][k] * b_s[k][c];
    __syncthreads();
  }
  C[c_off[t] + r * ldc + c] = acc;
}

}  // namespace

int launch_i8_tile_program(DeviceCtx* c, const int8_t* A, const int8_t* B, int32_t* C, int64_t lda, int64_t ldb,
                           int64_t ldc, int64_t n_tiles, const int64_t* d_c_off, const int64_t* d_term_begin,
                           const int64_t* d_a_off, const int64_t* d_b_off, cudaStream_t s) {
  (void)c;
  i8_tile_program_kernel<<<unsigned(n_tiles), 256, 0, s>>>(A, B, C, lda, ldb, ldc, d_c_off, d_term_begin, d_a_off,
                                                           d_b_off);
  count_launch();
  VT_CUDA(cudaGetLastError());
  return VT_OK;
}

}  // namespace vt
