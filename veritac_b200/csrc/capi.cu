// extern "C" entry points declared in include/veritac_b200.h: argument checking in the
// reference's plan domain, host<->device staging for host-pointer calls, launch, status.
#include <cstring>

#include "runtime.h"

using namespace vt;

namespace {

// The reference plan domain (validate_plan, specializations/gemmini_gemm/backend.py:121-136).
int check_i8_domain(int64_t M, int64_t N, int64_t K) {
  const int64_t d[3] = {M, N, K};
  const char* nm[3] = {"m", "n", "k"};
  for (int i = 0; i < 3; ++i) {
    if (d[i] < 16) return fail(VT_ERR_INVALID, "%s=%lld must be >= dim=16", nm[i], (long long)d[i]);
    if (d[i] % 16) return fail(VT_ERR_INVALID, "%s=%lld must be divisible by dim=16", nm[i], (long long)d[i]);
    if (d[i] > 0x7fffffffLL) return fail(VT_ERR_INVALID, "%s=%lld exceeds the 32-bit TMA extent", nm[i], (long long)d[i]);
  }
  if (K * 16384 > 2147483647LL)
    return fail(VT_ERR_INVALID, "overflow bound violated: k*16384 = %lld > 2147483647", (long long)(K * 16384));
  return VT_OK;
}

void raster_for(int raster, int batch_rows, int64_t M, int* mode, int* group) {
  switch (raster) {
    case VT_RASTER_BASELINE: *mode = 0; *group = 1; break;
    case VT_RASTER_REUSE_B: *mode = 1; *group = 1; break;
    case VT_RASTER_BATCHED: {
      // batch_rows 16-row Gemmini tiles live together = ceil(batch_rows*16 / 128) CTA tile-rows.
      const int64_t rows = int64_t(batch_rows < 1 ? 1 : batch_rows) * 16;
      *mode = 2;
      *group = int((rows + 127) / 128);
      break;
    }
    // VT_RASTER_AUTO: sweeps of 32 tile-rows of 128 (16 pair tiles): the rows of A of a sweep (32 MiB at K = 8192) stay
    // in L2 while B streams past once per sweep.  Measured at 8192^3, one process, 30-launch bursts, us per launch:
    // 16 tile-rows 358.7, 24 356.8, 32 354.6, 40 359.4, 48 369.4, 64 396-461, 8 378.7; the same order at
    // 16384 x 8192 x 4096 (389.2 / 383.3) and 8192 x 16384 x 8192 (711.7 / 705.0).
    default: *mode = 2; *group = 32; break;
  }
  (void)M;
}

// Two CTAs per tile need at least 256 rows to have work for both; below that one CTA per tile.  Products of more
// than one but at most two 256 x 256 tiles per CTA pair (a 1024-row shard of an 8192-wide product on 74 pairs) run
// as 256 x 512 tiles: the pair kernel's second wave of tiles would be its last, so there is no later tile whose MMAs
// the wide form's exposed epilogue could have overlapped, and its K loop runs closer to the tensor pipe's rate
// (measured 49.4 against 51.3 us at 1024 x 8192 x 8192; 96.8 against 98.1 at 2048 rows, 371 against 367 at 8192).
// 256 x 512 tiles where the 256 x 256 form would run a second round that most pairs take part in, on a long K:
// measured (K = 8192, whole tiles / wide, us) 128 tiles 49.8 / 48.8 and 47.5 / 47.0, 144 tiles 50.3 / 48.9 and
// 53.4 / 51.9; but 112 tiles 47.4 / 47.8, 96 tiles 48.2 / 51.8, 80 tiles 47.8 / 54.6 (the few pairs of a short
// second round run it fast, the wide form makes everybody's tile twice as long), and at K = 2048 128 tiles 21.8 / 22.2
// (the unoverlapped epilogue weighs more).
int resolve_i8_variant(int variant, int64_t M, int64_t N, int64_t K, int sm_count) {
  if (variant != VT_I8_AUTO) return variant;
  if (M <= 128) return VT_I8_B_AS_STORED;
  const int64_t tiles = ((M + 255) / 256) * ((N + 255) / 256);
  const int64_t pairs = sm_count / 2;
  return (tiles * 10 >= pairs * 17 && tiles <= 2 * pairs && N > 256 && K >= 4096) ? VT_I8_CTA_PAIR_WIDE : VT_I8_CTA_PAIR;
}

cudaStream_t pick_stream(DeviceCtx* c, void* stream) { return stream ? static_cast<cudaStream_t>(stream) : c->stream; }

// Host-pointer int8 GEMM, row blocks only: B and the first row block of A go in, then row blocks
// are computed while the next block of A streams in and the previous block of C streams out.
// With `b_ready` given, B is `dB` itself, already on the device once the work queued on that stream is done.
int i8gemm_from_host_rows(DeviceCtx* c, const int8_t* A, const int8_t* B, int32_t* C, int8_t* dA, const int8_t* dB,
                          int32_t* dC, int64_t M, int64_t N, int64_t K, int mode, int group, int variant,
                          const cudaStream_t* b_ready = nullptr) {
  // Row blocks: a multiple of 128 rows, at least 1024, about 8 blocks for large M.
  int64_t rows = ((M / 8 + 127) / 128) * 128;
  if (rows < 1024) rows = 1024;
  cudaEvent_t ev_b = c->ev[0], ev_in = c->ev[1], ev_k = c->ev[2];
  if (b_ready) {
    VT_CUDA(cudaEventRecord(ev_b, *b_ready));
  } else {
    VT_CUDA(cudaMemcpyAsync(const_cast<int8_t*>(dB), B, size_t(K) * N, cudaMemcpyHostToDevice, c->copy_in));
    VT_CUDA(cudaEventRecord(ev_b, c->copy_in));
  }
  VT_CUDA(cudaStreamWaitEvent(c->stream, ev_b, 0));
  for (int64_t r0 = 0; r0 < M; r0 += rows) {
    const int64_t r = (M - r0 < rows) ? (M - r0) : rows;
    VT_CUDA(cudaMemcpyAsync(dA + r0 * K, A + r0 * K, size_t(r) * K, cudaMemcpyHostToDevice, c->copy_in));
    VT_CUDA(cudaEventRecord(ev_in, c->copy_in));
    VT_CUDA(cudaStreamWaitEvent(c->stream, ev_in, 0));
    int rc = launch_i8gemm(c, dA + r0 * K, dB, dC + r0 * N, r, N, K, mode, group, variant, c->stream);
    if (rc) return rc;
    VT_CUDA(cudaEventRecord(ev_k, c->stream));
    VT_CUDA(cudaStreamWaitEvent(c->copy_out, ev_k, 0));
    VT_CUDA(cudaMemcpyAsync(C + r0 * N, dC + r0 * N, size_t(r) * N * sizeof(int32_t), cudaMemcpyDeviceToHost,
                            c->copy_out));
  }
  return VT_OK;
}

// Host-pointer int8 GEMM, growing corner: the output leaves over PCIe for twice as long as the
// operands take to arrive (4 bytes out per cell against 1 byte in per operand element), so the
// first cells of C must be ready long before B is complete.  A is cut into row blocks and B into
// column blocks; step s brings in column block s of B and row block s of A and computes the cells
// they complete: column block s of C for the rows already present, then row block s of C for the
// columns already present.  Each region goes out as soon as its kernel ends.  B's column blocks
// and C's regions are sub-matrices, copied as pitched 2-D transfers and addressed by the kernel
// through the row pitch of its tensor maps.
int i8gemm_from_host_corner(DeviceCtx* c, const int8_t* A, const int8_t* B, int32_t* C, int8_t* dA, int8_t* dB,
                            int32_t* dC, int64_t M, int64_t N, int64_t K, int mode, int group, int variant) {
  // Cut points in 32nds of the extent, rounded to whole 256-wide tiles: a small first corner so
  // that C starts to leave early, then few large regions (every region costs a launch and a copy;
  // measured on PCIe 5 x16 at 8192^3: 5.8 ms for these cuts, 6.35 ms for eight row blocks).
  const int cuts32[] = {4, 12, 20, 32};
  const int n_cuts = 4;
  int64_t rcut[4], ccut[4];
  int mb = 0, nb = 0;
  auto make_cuts = [&](int64_t extent, int64_t* cut) {
    int n = 0;
    int64_t last = 0;
    for (int i = 0; i < n_cuts; ++i) {
      int64_t x = (i + 1 == n_cuts) ? extent : ((extent * cuts32[i] / 32 + 255) / 256) * 256;
      if (x > extent) x = extent;
      if (x > last) cut[n++] = last = x;
    }
    return n;
  };
  mb = make_cuts(M, rcut);
  nb = make_cuts(N, ccut);
  const int steps = mb > nb ? mb : nb;
  cudaEvent_t ev_in = c->ev[1], ev_k = c->ev[2];
  auto compute_and_return = [&](int64_t r0, int64_t rows, int64_t c0, int64_t cols) -> int {
    VT_CUDA(cudaEventRecord(ev_in, c->copy_in));
    VT_CUDA(cudaStreamWaitEvent(c->stream, ev_in, 0));
    int rc = launch_i8gemm(c, dA + r0 * K, dB + c0, dC + r0 * N + c0, rows, cols, K, mode, group,
                           rows > 128 ? variant : int(VT_I8_B_AS_STORED), c->stream, N, N);
    if (rc) return rc;
    VT_CUDA(cudaEventRecord(ev_k, c->stream));
    VT_CUDA(cudaStreamWaitEvent(c->copy_out, ev_k, 0));
    VT_CUDA(cudaMemcpy2DAsync(C + r0 * N + c0, size_t(N) * 4, dC + r0 * N + c0, size_t(N) * 4, size_t(cols) * 4,
                              size_t(rows), cudaMemcpyDeviceToHost, c->copy_out));
    return VT_OK;
  };
  for (int s = 0; s < steps; ++s) {
    const int64_t rows_present = s == 0 ? 0 : (s < mb ? rcut[s - 1] : M);  // rows of A on the device before this step
    const int64_t cols_after = s < nb ? ccut[s] : N;                       // columns of B on the device after it
    if (s < nb) {
      const int64_t c0 = s == 0 ? 0 : ccut[s - 1], cols = ccut[s] - c0;
      VT_CUDA(cudaMemcpy2DAsync(dB + c0, size_t(N), B + c0, size_t(N), size_t(cols), size_t(K),
                                cudaMemcpyHostToDevice, c->copy_in));
      if (rows_present > 0) {
        int rc = compute_and_return(0, rows_present, c0, cols);
        if (rc) return rc;
      }
    }
    if (s < mb) {
      const int64_t r0 = s == 0 ? 0 : rcut[s - 1], rows = rcut[s] - r0;
      VT_CUDA(cudaMemcpyAsync(dA + r0 * K, A + r0 * K, size_t(rows) * K, cudaMemcpyHostToDevice, c->copy_in));
      int rc = compute_and_return(r0, rows, 0, cols_after);
      if (rc) return rc;
    }
  }
  return VT_OK;
}

// `b_ready`: B is a device pointer, valid once the work queued on that stream is done (the replicated operand of
// a row-sharded job); A and C are host pointers either way.
int i8gemm_from_host(DeviceCtx* c, const int8_t* A, const int8_t* B, int32_t* C, int64_t M, int64_t N, int64_t K,
                     int mode, int group, int variant, const cudaStream_t* b_ready = nullptr) {
  int8_t* dA = static_cast<int8_t*>(ctx_workspace(c, 0, size_t(M) * K));
  int8_t* dB = b_ready ? nullptr : static_cast<int8_t*>(ctx_workspace(c, 1, size_t(K) * N));
  int32_t* dC = static_cast<int32_t*>(ctx_workspace(c, 2, size_t(M) * N * sizeof(int32_t)));
  if (!dA || (!dB && !b_ready) || !dC) return VT_ERR_CUDA;
  int rc;
  if (b_ready)
    rc = i8gemm_from_host_rows(c, A, nullptr, C, dA, B, dC, M, N, K, mode, group, variant, b_ready);
  else if (M >= 2048 && N >= 2048)
    rc = i8gemm_from_host_corner(c, A, B, C, dA, dB, dC, M, N, K, mode, group, variant);
  else
    rc = i8gemm_from_host_rows(c, A, B, C, dA, dB, dC, M, N, K, mode, group, variant);
  if (rc) return rc;
  cudaEvent_t ev_done = c->ev[3];
  VT_CUDA(cudaEventRecord(ev_done, c->copy_out));
  VT_CUDA(cudaStreamWaitEvent(c->stream, ev_done, 0));
  return ctx_check_status(c, c->stream);
}

// Host-pointer fp32 GEMM on the 3xTF32 path, pipelined like the int8 one: B goes in whole and its lo
// part is written once; A then arrives in row blocks, and each block's lo pass, GEMM and the copy of
// its rows of C overlap the arrival of the next block.
int sgemm_tf32x3_from_host(DeviceCtx* c, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K) {
  int64_t rows = ((M / 8 + 255) / 256) * 256;
  if (rows < 512) rows = 512;
  float* dA = static_cast<float*>(ctx_workspace(c, 0, size_t(M) * K * 4));
  float* dB = static_cast<float*>(ctx_workspace(c, 1, size_t(K) * N * 4));
  float* dC = static_cast<float*>(ctx_workspace(c, 2, size_t(M) * N * 4));
  float* split = static_cast<float*>(ctx_workspace(c, 3, sgemm_tf32x3_workspace_bytes(rows, N, K)));
  if (!dA || !dB || !dC || !split) return VT_ERR_CUDA;
  cudaEvent_t ev_in = c->ev[1], ev_k = c->ev[2], ev_done = c->ev[3];
  VT_CUDA(cudaMemcpyAsync(dB, B, size_t(K) * N * 4, cudaMemcpyHostToDevice, c->copy_in));
  VT_CUDA(cudaEventRecord(ev_in, c->copy_in));
  VT_CUDA(cudaStreamWaitEvent(c->stream, ev_in, 0));
  int rc = launch_sgemm_tf32x3(c, dA, dB, dC, split, 0, N, K, c->stream, 2);   // B lo only
  if (rc) return rc;
  for (int64_t r0 = 0; r0 < M; r0 += rows) {
    const int64_t r = (M - r0 < rows) ? (M - r0) : rows;
    VT_CUDA(cudaMemcpyAsync(dA + r0 * K, A + r0 * K, size_t(r) * K * 4, cudaMemcpyHostToDevice, c->copy_in));
    VT_CUDA(cudaEventRecord(ev_in, c->copy_in));
    VT_CUDA(cudaStreamWaitEvent(c->stream, ev_in, 0));
    rc = launch_sgemm_tf32x3(c, dA + r0 * K, dB, dC + r0 * N, split, r, N, K, c->stream, 1);   // this block's A lo
    if (rc) return rc;
    VT_CUDA(cudaEventRecord(ev_k, c->stream));
    VT_CUDA(cudaStreamWaitEvent(c->copy_out, ev_k, 0));
    VT_CUDA(cudaMemcpyAsync(C + r0 * N, dC + r0 * N, size_t(r) * N * 4, cudaMemcpyDeviceToHost, c->copy_out));
  }
  VT_CUDA(cudaEventRecord(ev_done, c->copy_out));
  VT_CUDA(cudaStreamWaitEvent(c->stream, ev_done, 0));
  return ctx_check_status(c, c->stream);
}

// The automatic choice of fp32 kernel for device operands dA, dB, dC (only their alignment is looked at).
// Returns a VT_SGEMM_* value other than AUTO; VT_SGEMM_AUTO itself stands for "the FFMA tile kernels, whichever
// sgemm_tile_choice picks".
int choose_sgemm_variant(DeviceCtx* c, const float* dA, const float* dB, const float* dC, int64_t M, int64_t N, int64_t K) {
  const bool skinny_ok = M <= 16 && N % 4 == 0 &&
                         ((reinterpret_cast<uintptr_t>(dB) | reinterpret_cast<uintptr_t>(dC)) & 15) == 0;
  // The streaming kernels count arrivals per 128-wide slab in kTicketCount counters: more slabs than that go to
  // the tile kernels.
  const int64_t max_streamed = int64_t(kTicketCount) * 128;
  if (skinny_ok && N <= max_streamed && K >= 512 && (N >= 512 || (N >= 128 && double(N) * double(K) >= 1.0e6)))
    return VT_SGEMM_SKINNY_TF32X3;
  // Few rows against a large B: B is the traffic, and the row-panel kernel streams it once per 128 rows of A.
  // (measured against the tile kernels and the 3xTF32 pair kernel: ahead from 1 Mi elements of B up to 32 rows,
  // from 4 Mi up to 256 rows, from 16 Mi up to 384 rows).
  if (M > 16 && M <= 3 * SKINNY_UMMA_MAX_ROWS && N >= 128 && K >= 512 &&
      double(N) * double(K) >= (M <= 32 ? 1.0e6 : 4.0e6) && sgemm_skinny_umma_supported(dA, dB, dC, 1, N, K)) {
    // With few columns and a very long K every CTA holds a piece of the same few slabs, and one CTA per slab adds all
    // the partial tiles (128 x 128 x 65536: 148 of them, 0.15 ms, against 0.08 ms for the 32-wide FFMA kernel with
    // its own K split): the panel kernel's time is modelled as the stream of B (a panel of 16 rows at the rate of
    // the stream, one of 128 rows at half of it) plus that adding at 60 GB/s, and compared with the FFMA choice.
    double t_panel = 0;
    for (int64_t m0 = 0; m0 < M; m0 += SKINNY_UMMA_MAX_ROWS) {      // one launch per panel of up to 128 rows
      const int64_t rows = M - m0 < SKINNY_UMMA_MAX_ROWS ? M - m0 : SKINNY_UMMA_MAX_ROWS;
      int ctas, slabs, max_parts;
      sgemm_skinny_umma_plan(rows, N, K, c->sm_count, &ctas, &slabs, &max_parts);
      const double stream = double(K) * double(N) * 4.0 / 5.0e12 * (1.0 + (rows > 16 ? double(rows - 16) / 112.0 : 0.0));
      const double adding = max_parts > 1 ? double(max_parts) * double(rows) * 512.0 / 6.0e10 : 0.0;
      t_panel += 6.0e-6 + stream + adding;
    }
    int tile_variant;
    if (t_panel < sgemm_tile_choice(c, dA, dB, dC, M, N, K, &tile_variant))
      return VT_SGEMM_PANEL_TF32X3;
  }
  // Few columns against a large A: the mirror image (measured ahead of the tile kernels and the 3xTF32 pair kernel
  // from 4 Mi elements of A up to 32 columns, from 12 Mi up to 64, from 16 Mi up to 128).
  if (N <= SKINNY_UMMA_MAX_ROWS && K >= 256 &&
      double(M) * double(K) >= (N <= 32 ? 4.0e6 : N <= 64 ? 1.2e7 : 1.6e7) && sgemm_tall_umma_supported(dA, dB, dC, M, N, K))
    return VT_SGEMM_TALL_TF32X3;
  // Two panels of 128 columns against a very large A: still ahead of the pair kernel (8192 x 256 x 8192: 0.294
  // against 0.326 ms).
  if (N <= 2 * SKINNY_UMMA_MAX_ROWS && K >= 256 && double(M) * double(K) >= 6.4e7 &&
      sgemm_tall_umma_supported(dA, dB, dC, M, N, K))
    return VT_SGEMM_TALL_TF32X3;
  // Products of 0.1 GFLOP and more go to the tensor cores (3xTF32, measured ~1e-6 relative Frobenius error at any K)
  // when the model says that is faster than the best FFMA kernel.  Its time is modelled as two launches (6 us), the pass that
  // writes the lo parts and the write of C (8 bytes per element of A and B, 4 per element of C, at ~5.5 TB/s) and
  // K x 29 ns for every wave of 256x256 tiles over the 74 CTA pairs (measured on cubes of 896 to 1536, which is where
  // the comparison is close; at 8192^3, under the power cap, a wave takes K x 34 ns).  (A fixed floor of 0.5 GFLOP and a 10 % margin
  // in favour of FFMA were dropped after an audit on 80 random mid-sized shapes: with them 596 x 2504 x 252 ran at 33.9 us
  // against 18.1, and four shapes of 1-4 GFLOP 10-20 % behind.)
  if (M >= 128 && N >= 16 && K >= 64 && double(M) * double(N) * double(K) >= 1.0e8 &&
      sgemm_tf32x3_supported(dA, dB, dC, M, N, K)) {
    int tile_variant;
    const double t_tile = sgemm_tile_choice(c, dA, dB, dC, M, N, K, &tile_variant);
    const double pair_tiles = double((M + 255) / 256) * double((N + 255) / 256);
    const double pairs = c->sm_count / 2;
    const double waves = pair_tiles <= pairs ? 1.0 : double(int64_t((pair_tiles + pairs - 1) / pairs));
    const double t_tc = 6.0e-6 + ((double(M) * K + double(K) * N) * 8.0 + double(M) * N * 4.0) / 5.5e12 +
                        waves * double(K) * 2.9e-8;
    if (t_tc < t_tile) return VT_SGEMM_TF32X3;
  }
  return VT_SGEMM_AUTO;
}

}  // namespace

extern "C" {

int vt_device_count(void) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDeviceCount");
  return n;
}

const char* vt_last_error(void) { return last_error_text(); }

int vt_i8gemm(int dev, const int8_t* A, const int8_t* B, int32_t* C, int64_t M, int64_t N, int64_t K, int raster,
              int batch_rows, int variant, int where, void* stream) {
  clear_error_text();
  if (!A || !B || !C) return fail(VT_ERR_INVALID, "null operand");
  if (where != VT_HOST && where != VT_DEVICE && where != VT_HOST_AC_DEVICE_B)
    return fail(VT_ERR_INVALID, "where must be VT_HOST, VT_DEVICE or VT_HOST_AC_DEVICE_B");
  if (raster < VT_RASTER_BASELINE || raster > VT_RASTER_AUTO) return fail(VT_ERR_INVALID, "unknown raster %d", raster);
  if (raster == VT_RASTER_BATCHED && (batch_rows < 1 || batch_rows > 64))
    return fail(VT_ERR_INVALID, "batch_rows must be in 1..64 (accumulator rows 16..1024)");
  int rc = check_i8_domain(M, N, K);
  if (rc) return rc;
  DeviceCtx* c = ctx_for(dev);
  if (!c) return VT_ERR_CUDA;
  int mode, group;
  raster_for(raster, batch_rows, M, &mode, &group);
  variant = resolve_i8_variant(variant, M, N, K, c->sm_count);
  if (where == VT_HOST) return i8gemm_from_host(c, A, B, C, M, N, K, mode, group, variant);
  if (where == VT_HOST_AC_DEVICE_B) {
    const cudaStream_t b_ready = pick_stream(c, stream);
    return i8gemm_from_host(c, A, B, C, M, N, K, mode, group, variant, &b_ready);
  }
  return launch_i8gemm(c, A, B, C, M, N, K, mode, group, variant, pick_stream(c, stream));
}

int vt_i8_stage_b_block(int dev, int8_t* dst, const int8_t* B_host, int64_t K, int64_t N, int64_t c0, int64_t cols,
                        void* stream) {
  clear_error_text();
  if (!dst || !B_host) return fail(VT_ERR_INVALID, "null operand");
  if (K < 1 || N < 1 || c0 < 0 || cols < 1 || c0 + cols > N) return fail(VT_ERR_INVALID, "column block outside B");
  DeviceCtx* c = ctx_for(dev);
  if (!c) return VT_ERR_CUDA;
  VT_CUDA(cudaMemcpy2DAsync(dst, size_t(cols), B_host + c0, size_t(N), size_t(cols), size_t(K), cudaMemcpyHostToDevice,
                            pick_stream(c, stream)));
  return VT_OK;
}

int vt_i8gemm_rows_streamed_b(int dev, const int8_t* A, int a_where, const int8_t* const* B_blocks,
                              const int64_t* block_cols, void* const* block_ready, int n_blocks, int32_t* C, int64_t M,
                              int64_t N, int64_t K, int raster, int batch_rows, int variant) {
  clear_error_text();
  if (a_where != VT_HOST && a_where != VT_DEVICE) return fail(VT_ERR_INVALID, "a_where must be VT_HOST or VT_DEVICE");
  if (!A || !B_blocks || !block_cols || !block_ready || !C) return fail(VT_ERR_INVALID, "null operand");
  if (n_blocks < 1 || n_blocks > 64) return fail(VT_ERR_INVALID, "n_blocks must be in 1..64");
  if (raster < VT_RASTER_BASELINE || raster > VT_RASTER_AUTO) return fail(VT_ERR_INVALID, "unknown raster %d", raster);
  if (raster == VT_RASTER_BATCHED && (batch_rows < 1 || batch_rows > 64))
    return fail(VT_ERR_INVALID, "batch_rows must be in 1..64 (accumulator rows 16..1024)");
  int rc = check_i8_domain(M, N, K);
  if (rc) return rc;
  int64_t total = 0;
  for (int j = 0; j < n_blocks; ++j) {
    if (!B_blocks[j] || !block_ready[j]) return fail(VT_ERR_INVALID, "null block %d", j);
    rc = check_i8_domain(M, block_cols[j], K);
    if (rc) return rc;
    total += block_cols[j];
  }
  if (total != N) return fail(VT_ERR_INVALID, "block widths add up to %lld, not N = %lld", (long long)total, (long long)N);
  DeviceCtx* c = ctx_for(dev);
  if (!c) return VT_ERR_CUDA;
  int mode, group;
  raster_for(raster, batch_rows, M, &mode, &group);
  const int8_t* dA = A;
  int32_t* dC = static_cast<int32_t*>(ctx_workspace(c, 2, size_t(M) * N * sizeof(int32_t)));
  if (!dC) return VT_ERR_CUDA;
  cudaEvent_t ev_in = c->ev[1], ev_k = c->ev[2], ev_done = c->ev[3];
  if (a_where == VT_HOST) {
    int8_t* wa = static_cast<int8_t*>(ctx_workspace(c, 0, size_t(M) * K));
    if (!wa) return VT_ERR_CUDA;
    VT_CUDA(cudaMemcpyAsync(wa, A, size_t(M) * K, cudaMemcpyHostToDevice, c->copy_in));
    VT_CUDA(cudaEventRecord(ev_in, c->copy_in));
    VT_CUDA(cudaStreamWaitEvent(c->stream, ev_in, 0));
    dA = wa;
  }
  int64_t c0 = 0;
  for (int j = 0; j < n_blocks; ++j) {
    const int64_t cols = block_cols[j];
    VT_CUDA(cudaStreamWaitEvent(c->stream, static_cast<cudaEvent_t>(block_ready[j]), 0));
    rc = launch_i8gemm(c, dA, B_blocks[j], dC + c0, M, cols, K, mode, group, resolve_i8_variant(variant, M, cols, K, c->sm_count),
                       c->stream, cols, N);
    if (rc) return rc;
    VT_CUDA(cudaEventRecord(ev_k, c->stream));
    VT_CUDA(cudaStreamWaitEvent(c->copy_out, ev_k, 0));
    VT_CUDA(cudaMemcpy2DAsync(C + c0, size_t(N) * 4, dC + c0, size_t(N) * 4, size_t(cols) * 4, size_t(M),
                              cudaMemcpyDeviceToHost, c->copy_out));
    c0 += cols;
  }
  VT_CUDA(cudaEventRecord(ev_done, c->copy_out));
  VT_CUDA(cudaStreamWaitEvent(c->stream, ev_done, 0));
  return ctx_check_status(c, c->stream);
}

int vt_i8gemm_shared_b(int dev, const int8_t* A, const int8_t* B, int32_t* C, int64_t batch, int64_t M, int64_t N,
                       int64_t K, int acc_rows, int where, void* stream) {
  clear_error_text();
  if (batch < 1) return fail(VT_ERR_INVALID, "batch must be positive");
  if (acc_rows < 16 || acc_rows > 1024 || acc_rows % 16)
    return fail(VT_ERR_INVALID, "accumulator_rows=%d must be a multiple of 16 in 16..1024", acc_rows);
  int rc = check_i8_domain(M, N, K);
  if (rc) return rc;
  if (batch * M > 0x7fffffffLL) return fail(VT_ERR_INVALID, "batch*M exceeds the 32-bit TMA extent");
  // One A_i never shares an output row with another, and M is a multiple of 16, so the stacked
  // (batch*M) x K matrix against B is exactly the batch of products; B is fetched once per
  // column sweep for all A_i that are resident together.
  return vt_i8gemm(dev, A, B, C, batch * M, N, K, VT_RASTER_BATCHED, acc_rows / 16 > 64 ? 64 : acc_rows / 16,
                   VT_I8_AUTO, where, stream);
}

int vt_i8_tile_program(int dev, const int8_t* A, int64_t a_elems, const int8_t* B, int64_t b_elems, int32_t* C,
                       int64_t c_elems, int64_t lda, int64_t ldb, int64_t ldc, int64_t n_tiles,
                       const int64_t* c_off, const int64_t* term_begin, const int64_t* a_off,
                       const int64_t* b_off, int where, void* stream) {
  clear_error_text();
  if (!A || !B || !C || !c_off || !term_begin) return fail(VT_ERR_INVALID, "null operand");
  if (where != VT_HOST && where != VT_DEVICE) return fail(VT_ERR_INVALID, "where must be VT_HOST or VT_DEVICE");
  if (n_tiles < 1 || n_tiles > 0x7fffffffLL) return fail(VT_ERR_PROGRAM, "tile count out of range");
  // Operand strides are the stream's config_ld strides: 0 repeats one row, 1..15 makes rows overlap (the reference
  // interpreter takes any stride >= 0); output tiles must not fold onto themselves.
  if (lda < 0 || ldb < 0) return fail(VT_ERR_PROGRAM, "operand row strides must be >= 0");
  if (ldc < 16) return fail(VT_ERR_PROGRAM, "output row stride must be >= 16");
  if (term_begin[0] != 0) return fail(VT_ERR_PROGRAM, "term_begin[0] must be 0");
  const int64_t n_terms = term_begin[n_tiles];
  if (n_terms > 0 && (!a_off || !b_off)) return fail(VT_ERR_INVALID, "null term arrays");
  for (int64_t t = 0; t < n_tiles; ++t) {
    const int64_t cnt = term_begin[t + 1] - term_begin[t];
    if (cnt < 0) return fail(VT_ERR_PROGRAM, "term_begin must be non-decreasing");
    if (cnt > 8191) return fail(VT_ERR_OVERFLOW, "tile %lld sums %lld products; more than 8191 can leave int32",
                                (long long)t, (long long)cnt);
    if (c_off[t] < 0 || c_off[t] + 15 * ldc + 16 > c_elems) return fail(VT_ERR_PROGRAM, "output tile %lld out of bounds", (long long)t);
  }
  for (int64_t j = 0; j < n_terms; ++j) {
    if (a_off[j] < 0 || a_off[j] + 15 * lda + 16 > a_elems) return fail(VT_ERR_PROGRAM, "A tile of term %lld out of bounds", (long long)j);
    if (b_off[j] < 0 || b_off[j] + 15 * ldb + 16 > b_elems) return fail(VT_ERR_PROGRAM, "B tile of term %lld out of bounds", (long long)j);
  }
  DeviceCtx* c = ctx_for(dev);
  if (!c) return VT_ERR_CUDA;
  cudaStream_t s = where == VT_HOST ? c->stream : pick_stream(c, stream);

  // Program tables: packed into the context's pinned staging block (grow-only, reused once the previous upload
  // from it has been consumed), then one asynchronous upload into workspace slot 3.  Nothing here waits for the
  // caller's stream.
  const size_t n_c = size_t(n_tiles), n_tb = size_t(n_tiles) + 1, n_t = size_t(n_terms);
  const size_t table_elems = n_c + n_tb + 2 * n_t;
  int64_t* packed = static_cast<int64_t*>(ctx_pinned_staging(c, table_elems * 8));
  if (!packed) return VT_ERR_CUDA;
  std::memcpy(packed, c_off, n_c * 8);
  std::memcpy(packed + n_c, term_begin, n_tb * 8);
  if (n_t) {
    std::memcpy(packed + n_c + n_tb, a_off, n_t * 8);
    std::memcpy(packed + n_c + n_tb + n_t, b_off, n_t * 8);
  }
  int64_t* d_tab = static_cast<int64_t*>(ctx_workspace(c, 3, table_elems * 8));
  if (!d_tab) return VT_ERR_CUDA;
  VT_CUDA(cudaMemcpyAsync(d_tab, packed, table_elems * 8, cudaMemcpyHostToDevice, s));
  VT_CUDA(cudaEventRecord(c->staging_consumed, s));

  const int8_t* dA = A;
  const int8_t* dB = B;
  int32_t* dC = C;
  if (where == VT_HOST) {
    int8_t* wa = static_cast<int8_t*>(ctx_workspace(c, 0, size_t(a_elems)));
    int8_t* wb = static_cast<int8_t*>(ctx_workspace(c, 1, size_t(b_elems)));
    int32_t* wc = static_cast<int32_t*>(ctx_workspace(c, 2, size_t(c_elems) * 4));
    if (!wa || !wb || !wc) return VT_ERR_CUDA;
    VT_CUDA(cudaMemcpyAsync(wa, A, size_t(a_elems), cudaMemcpyHostToDevice, s));
    VT_CUDA(cudaMemcpyAsync(wb, B, size_t(b_elems), cudaMemcpyHostToDevice, s));
    // Cells no tile covers keep the caller's contents.
    VT_CUDA(cudaMemcpyAsync(wc, C, size_t(c_elems) * 4, cudaMemcpyHostToDevice, s));
    dA = wa; dB = wb; dC = wc;
  }
  int rc = launch_i8_tile_program(c, dA, dB, dC, lda, ldb, ldc, n_tiles, d_tab, d_tab + n_c, d_tab + n_c + n_tb,
                                  d_tab + n_c + n_tb + n_t, s);
  if (rc) return rc;
  if (where == VT_HOST) {
    VT_CUDA(cudaMemcpyAsync(C, dC, size_t(c_elems) * 4, cudaMemcpyDeviceToHost, s));
    return ctx_check_status(c, s);
  }
  return VT_OK;
}

int vt_sgemm(int dev, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int variant,
             int where, void* stream) {
  clear_error_text();
  if (!A || !B || !C) return fail(VT_ERR_INVALID, "null operand");
  if (where != VT_HOST && where != VT_DEVICE) return fail(VT_ERR_INVALID, "where must be VT_HOST or VT_DEVICE");
  if (M < 1 || N < 1 || K < 1) return fail(VT_ERR_INVALID, "dimensions must be positive");
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return fail(VT_ERR_INVALID, "dimension overflows int");
  if (variant < VT_SGEMM_AUTO || variant > VT_SGEMM_PIPE64X128) return fail(VT_ERR_INVALID, "unknown sgemm variant %d", variant);
  DeviceCtx* c = ctx_for(dev);
  if (!c) return VT_ERR_CUDA;
  cudaStream_t s = where == VT_HOST ? c->stream : pick_stream(c, stream);

  // Large host-buffer products on the tensor-core path are pipelined against the PCIe copies.
  if (where == VT_HOST && (variant == VT_SGEMM_AUTO || variant == VT_SGEMM_TF32X3) && M >= 1024 && N >= 256 && K >= 256 &&
      double(M) * double(N) * double(K) >= 5.0e8 && N % 4 == 0 && K % 4 == 0)
    return sgemm_tf32x3_from_host(c, A, B, C, M, N, K);

  const float* dA = A;
  const float* dB = B;
  float* dC = C;
  if (where == VT_HOST) {
    float* wa = static_cast<float*>(ctx_workspace(c, 0, size_t(M) * K * 4));
    float* wb = static_cast<float*>(ctx_workspace(c, 1, size_t(K) * N * 4));
    float* wc = static_cast<float*>(ctx_workspace(c, 2, size_t(M) * N * 4));
    if (!wa || !wb || !wc) return VT_ERR_CUDA;
    VT_CUDA(cudaMemcpyAsync(wa, A, size_t(M) * K * 4, cudaMemcpyHostToDevice, s));
    VT_CUDA(cudaMemcpyAsync(wb, B, size_t(K) * N * 4, cudaMemcpyHostToDevice, s));
    dA = wa; dB = wb; dC = wc;
  }
  const bool skinny_ok = M <= 16 && N % 4 == 0 &&
                         ((reinterpret_cast<uintptr_t>(dB) | reinterpret_cast<uintptr_t>(dC)) & 15) == 0;
  if (variant == VT_SGEMM_AUTO) {
    // The choice is a few models' worth of arithmetic, which a 5 us launch feels: the last shapes asked about on
    // this device are remembered (with the alignment of their operands, which some kernels depend on).
    const uint32_t align = uint32_t((reinterpret_cast<uintptr_t>(dA) | reinterpret_cast<uintptr_t>(dB) |
                                     reinterpret_cast<uintptr_t>(dC)) & 15);
    DeviceCtx::Choice* hit = nullptr;
    for (auto& e : c->sgemm_choices)
      if (e.variant != 0 && e.M == M && e.N == N && e.K == K && e.align == align) hit = &e;
    if (hit) {
      variant = hit->variant;
    } else {
      variant = choose_sgemm_variant(c, dA, dB, dC, M, N, K);
      if (variant == VT_SGEMM_AUTO) sgemm_tile_choice(c, dA, dB, dC, M, N, K, &variant);
      DeviceCtx::Choice& slot = c->sgemm_choices[c->sgemm_choice_next++ % 8];
      slot.M = M; slot.N = N; slot.K = K; slot.align = align; slot.variant = variant;
    }
  }
  int rc;
  if (variant == VT_SGEMM_TALL_TF32X3) {
    if (!sgemm_tall_umma_supported(dA, dB, dC, M, N, K))
      return fail(VT_ERR_UNSUPPORTED, "tall tensor-core kernel needs N %% 4 == 0, K %% 4 == 0 and 16-byte aligned A and C");
    // Panels of up to 128 columns, one launch each, in stream order: the scratch (partial tiles, then [B | B lo])
    // and the tickets are reused.
    size_t pbytes = 0, cat_bytes = 0;
    for (int64_t n0 = 0; n0 < N; n0 += SKINNY_UMMA_MAX_ROWS) {
      const int64_t width = N - n0 < SKINNY_UMMA_MAX_ROWS ? N - n0 : SKINNY_UMMA_MAX_ROWS;
      int max_parts;
      size_t cat;
      sgemm_tall_umma_plan(M, width, K, c->sm_count, &max_parts, &cat);
      const size_t need = max_parts > 1 ? size_t(max_parts) * size_t(M) * size_t(width) * 4 : 0;
      if (need > pbytes) pbytes = need;
      if (cat > cat_bytes) cat_bytes = cat;
    }
    pbytes = (pbytes + 255) & ~size_t(255);
    float* scratch = static_cast<float*>(ctx_workspace(c, 3, pbytes + cat_bytes));
    if (!scratch) return VT_ERR_CUDA;
    rc = VT_OK;
    for (int64_t n0 = 0; n0 < N && rc == VT_OK; n0 += SKINNY_UMMA_MAX_ROWS) {
      const int64_t width = N - n0 < SKINNY_UMMA_MAX_ROWS ? N - n0 : SKINNY_UMMA_MAX_ROWS;
      rc = launch_sgemm_tall_umma(c, dA, dB + n0, dC + n0, pbytes ? scratch : nullptr, c->tickets, scratch + pbytes / 4, M,
                                  width, K, N, N, s);
    }
  } else if (variant == VT_SGEMM_PANEL_TF32X3) {
    if (!sgemm_skinny_umma_supported(dA, dB, dC, 1, N, K))
      return fail(VT_ERR_UNSUPPORTED, "row-panel kernel needs N %% 4 == 0, K %% 4 == 0 and 16-byte aligned operands");
    size_t pbytes = 0;
    for (int64_t m0 = 0; m0 < M; m0 += SKINNY_UMMA_MAX_ROWS) {
      const int64_t rows = M - m0 < SKINNY_UMMA_MAX_ROWS ? M - m0 : SKINNY_UMMA_MAX_ROWS;
      int ctas, slabs, max_parts;
      sgemm_skinny_umma_plan(rows, N, K, c->sm_count, &ctas, &slabs, &max_parts);
      const size_t need = max_parts > 1 ? size_t(max_parts) * size_t(rows) * size_t(N) * 4 : 0;
      if (need > pbytes) pbytes = need;
    }
    float* partials = nullptr;
    if (pbytes) {
      partials = static_cast<float*>(ctx_workspace(c, 3, pbytes));
      if (!partials) return VT_ERR_CUDA;
    }
    rc = VT_OK;
    // One launch per panel, in stream order: the partial tiles and the tickets are reused.
    for (int64_t m0 = 0; m0 < M && rc == VT_OK; m0 += SKINNY_UMMA_MAX_ROWS) {
      const int64_t rows = M - m0 < SKINNY_UMMA_MAX_ROWS ? M - m0 : SKINNY_UMMA_MAX_ROWS;
      rc = launch_sgemm_skinny_umma(c, dA + m0 * K, dB, dC + m0 * N, partials, c->tickets, rows, N, K, s);
    }
  } else if (variant == VT_SGEMM_SKINNY_TF32X3 || variant == VT_SGEMM_SKINNY_MMA_SYNC) {
    if (!skinny_ok) return fail(VT_ERR_UNSUPPORTED, "skinny kernel needs M <= 16, N %% 4 == 0 and 16-byte aligned B, C");
    const bool umma = variant == VT_SGEMM_SKINNY_TF32X3 && sgemm_skinny_umma_supported(dA, dB, dC, M, N, K);
    int ctas, slabs, max_parts;
    if (umma) sgemm_skinny_umma_plan(M, N, K, c->sm_count, &ctas, &slabs, &max_parts);
    else sgemm_skinny_tma_plan(N, K, c->sm_count, &ctas, &slabs, &max_parts);
    float* partials = nullptr;
    if (max_parts > 1) {
      partials = static_cast<float*>(ctx_workspace(c, 3, size_t(max_parts) * size_t(M) * size_t(N) * 4));
      if (!partials) return VT_ERR_CUDA;
    }
    rc = umma ? launch_sgemm_skinny_umma(c, dA, dB, dC, partials, c->tickets, M, N, K, s)
              : launch_sgemm_skinny_tma(c, dA, dB, dC, partials, c->tickets, M, N, K, s);
  } else if (variant == VT_SGEMM_SKINNY) {
    if (!skinny_ok) return fail(VT_ERR_UNSUPPORTED, "skinny kernel needs M <= 16, N %% 4 == 0 and 16-byte aligned B, C");
    int ksplit = 1;
    const size_t pbytes = sgemm_skinny_partials_bytes(M, N, K, c->sm_count, &ksplit);
    float* partials = nullptr;
    if (pbytes) {
      partials = static_cast<float*>(ctx_workspace(c, 3, pbytes));
      if (!partials) return VT_ERR_CUDA;
    }
    rc = launch_sgemm_skinny(c, dA, dB, dC, partials, M, N, K, ksplit, s);
  } else if (variant == VT_SGEMM_TF32X3) {
    if (!sgemm_tf32x3_supported(dA, dB, dC, M, N, K))
      return fail(VT_ERR_UNSUPPORTED, "3xTF32 kernel needs N %% 4 == 0, K %% 4 == 0 and 16-byte aligned operands");
    float* split = static_cast<float*>(ctx_workspace(c, 3, sgemm_tf32x3_workspace_bytes(M, N, K)));
    if (!split) return VT_ERR_CUDA;
    rc = launch_sgemm_tf32x3(c, dA, dB, dC, split, M, N, K, s);
  } else {
    rc = launch_sgemm(c, dA, dB, dC, M, N, K, variant, s);
  }
  if (rc) return rc;
  if (where == VT_HOST) {
    VT_CUDA(cudaMemcpyAsync(C, dC, size_t(M) * N * 4, cudaMemcpyDeviceToHost, s));
    return ctx_check_status(c, s);
  }
  return VT_OK;
}

int vt_sgemm_auto_variant(int dev, int64_t M, int64_t N, int64_t K) {
  clear_error_text();
  if (M < 1 || N < 1 || K < 1) return fail(VT_ERR_INVALID, "dimensions must be positive");
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return fail(VT_ERR_INVALID, "dimension overflows int");
  // A question, not a launch: the caller's current device is put back.
  struct Restore {
    int prev = -1;
    Restore() { if (cudaGetDevice(&prev) != cudaSuccess) prev = -1; }
    ~Restore() { if (prev >= 0) cudaSetDevice(prev); }
  } restore;
  DeviceCtx* c = ctx_for(dev);
  if (!c) return VT_ERR_CUDA;
  const float* aligned = reinterpret_cast<const float*>(uintptr_t(256));   // never dereferenced
  int variant = choose_sgemm_variant(c, aligned, aligned, aligned, M, N, K);
  if (variant == VT_SGEMM_AUTO) sgemm_tile_choice(c, aligned, aligned, aligned, M, N, K, &variant);
  return variant;
}

int vt_test_set_wait_hooks(int dev, int64_t wait_limit_cycles, int i8_stop_fill) {
  clear_error_text();
  DeviceCtx* c = ctx_for(dev);
  if (!c) return VT_ERR_CUDA;
  c->wait_limit_cycles = wait_limit_cycles > 0 ? (long long)wait_limit_cycles : 4000000000LL;
  c->i8_stop_fill = i8_stop_fill < 0 ? -1 : i8_stop_fill;
  return VT_OK;
}

int vt_test_set_sgemm_splits(int dev, int splits) {
  clear_error_text();
  DeviceCtx* c = ctx_for(dev);
  if (!c) return VT_ERR_CUDA;
  c->sgemm_force_splits = splits;
  return VT_OK;
}

int vt_test_expire_wait(int dev, void* stream) {
  clear_error_text();
  DeviceCtx* c = ctx_for(dev);
  if (!c) return VT_ERR_CUDA;
  return launch_expire_wait(c, pick_stream(c, stream));
}

int vt_sync(int dev, void* stream) {
  clear_error_text();
  DeviceCtx* c = ctx_for(dev);
  if (!c) return VT_ERR_CUDA;
  cudaStream_t s = pick_stream(c, stream);
  VT_CUDA(cudaStreamSynchronize(s));
  return ctx_check_status(c, s);
}

void* vt_host_alloc(size_t bytes) {
  clear_error_text();
  void* p = nullptr;
  cudaError_t e = cudaMallocHost(&p, bytes ? bytes : 1);
  if (e != cudaSuccess) {
    fail_cuda(e, "cudaMallocHost");
    return nullptr;
  }
  return p;
}

int vt_host_free(void* p) {
  clear_error_text();
  if (!p) return VT_OK;
  VT_CUDA(cudaFreeHost(p));
  return VT_OK;
}

int64_t vt_launch_count(void) { return launch_count(); }

int vt_shutdown(void) {
  clear_error_text();
  ctx_destroy_all();
  return VT_OK;
}

}  // extern "C"
