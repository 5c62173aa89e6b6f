// Host-side runtime shared by the kernels' launchers and the C-ABI: per-device context (stream,
// status word, grow-only workspace), error reporting, the driver entry point used to encode TMA
// tensor maps, and the launch counter that the benchmark reports.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>

#include "../../include/veritac_b200.h"

namespace vt {

constexpr int kTicketCount = 4096;

struct DeviceCtx {
  int dev = -1;
  std::atomic<bool> ready{false};
  int sm_count = 0;
  size_t smem_optin = 0;
  cudaStream_t stream = nullptr;       // library-owned stream used when the caller passes none
  cudaStream_t copy_in = nullptr;      // host->device staging for the host-pointer entry points
  cudaStream_t copy_out = nullptr;     // device->host staging
  int* status = nullptr;               // device word kernels write a KSTAT_* code into
  int* status_host = nullptr;          // pinned mirror
  int* tickets = nullptr;              // kTicketCount zeroed counters (arrivals per slab of the skinny kernels, per tile of a K split)
  // Test hooks (vt_test_set_wait_hooks): how long a device-side wait may take, and the ring fill at which the odd
  // CTA of every int8 pair stops (-1: never).
  long long wait_limit_cycles = 4000000000LL;
  int i8_stop_fill = -1;
  // pipelined FFMA kernel: clusters of 1..8 CTAs of each tile shape the device holds at once (filled on first use)
  int ffma_capacity[3][9] = {};
  bool ffma_capacity_known = false;
  // the automatic fp32 choice for the last eight (shape, operand alignment) combinations asked about
  struct Choice { int64_t M = 0, N = 0, K = 0; uint32_t align = 0; int variant = 0; };
  Choice sgemm_choices[8];
  unsigned sgemm_choice_next = 0;
  int sgemm_force_splits = 0;          // test hook (vt_test_set_sgemm_splits): K split of the FFMA tile kernels, 0 = automatic
  // grow-only device workspace for host-pointer calls and operand re-layouts
  void* ws[4] = {nullptr, nullptr, nullptr, nullptr};
  size_t ws_bytes[4] = {0, 0, 0, 0};
  cudaEvent_t ev[8] = {};
  // pinned host block for small tables that go to the device asynchronously (tile programs)
  void* staging = nullptr;
  size_t staging_bytes = 0;
  cudaEvent_t staging_consumed = nullptr;   // recorded after the last upload from `staging`
  uint32_t func_attr_mask = 0;         // which kernels already had their shared-memory opt-in set here
};

// Error text for the calling thread; returns `code` so call sites can `return fail(...)`.
int fail(int code, const char* fmt, ...);
int fail_cuda(cudaError_t e, const char* what);
const char* last_error_text();
void clear_error_text();
long long launch_count();
void ctx_destroy_all();

// Makes `dev` current and returns its context, creating it on first use; nullptr + error set on failure.
DeviceCtx* ctx_for(int dev);
// Grow-only workspace slot; returns nullptr (error set) on allocation failure.
void* ctx_workspace(DeviceCtx* c, int slot, size_t bytes);
// The context's pinned staging block, at least `bytes` long, free to overwrite (waits for the upload that last
// read it); nullptr + error set on failure.
void* ctx_pinned_staging(DeviceCtx* c, size_t bytes);
// Reads and clears the device status word after the stream has drained.
int ctx_check_status(DeviceCtx* c, cudaStream_t s);
void count_launch(int n = 1);

// cuTensorMapEncodeTiled for a row-major 2-D byte/word matrix: `inner` contiguous elements per
// row, `outer` rows, 128-byte swizzle, zero fill outside the matrix.
int encode_tmap_2d(CUtensorMap* out, CUtensorMapDataType dtype, int elem_bytes, const void* base, uint64_t inner,
                   uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner, uint32_t box_outer,
                   CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B);

#define VT_CUDA(expr)                                   \
  do {                                                  \
    cudaError_t _e = (expr);                            \
    if (_e != cudaSuccess) return vt::fail_cuda(_e, #expr); \
  } while (0)

// Launches `kernel` so that its set-up may overlap the tail of the kernel before it on the stream
// (programmatic stream serialization).  The kernel must call grid_dependency_wait() (ptx_sm100.cuh) before
// it touches global memory.
template <class... KArgs, class... Args>
cudaError_t launch_overlapped(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t s,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel that runs in thread-block clusters of `cluster` consecutive CTAs (grid a multiple of it).
template <class... KArgs, class... Args>
cudaError_t launch_overlapped_cluster(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem,
                                      unsigned cluster, cudaStream_t s, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- kernel launchers (device pointers only) ------------------------------------------------
// raster_mode: 0 row-major tiles, 1 column-major tiles, 2 grouped (group = tile-rows per sweep).
// variant: VT_I8_B_AS_STORED (one CTA per 128 x 256 tile), VT_I8_CTA_PAIR (two CTAs per 256 x 256 tile),
// VT_I8_CTA_PAIR_WIDE (two CTAs per 256 x 512 tile).
// ldb / ldc: row pitch of B and C in elements when they are sub-blocks of wider matrices (0 = N).
int launch_i8gemm(DeviceCtx* c, const int8_t* A, const int8_t* B, int32_t* C, int64_t M, int64_t N, int64_t K,
                  int raster_mode, int group, int variant, cudaStream_t s, int64_t ldb = 0, int64_t ldc = 0);
// VT_I8_CTA_PAIR_WIDE: CTA pairs on 256 x 512 tiles (i8gemm_wide_sm100.cu); launch_i8gemm forwards to it.
int launch_i8gemm_wide(DeviceCtx* c, const int8_t* A, const int8_t* B, int32_t* C, int64_t M, int64_t N, int64_t K,
                       int raster_mode, int group, cudaStream_t s, int64_t ldb, int64_t ldc);
// Test hook: one CTA whose bounded wait runs out (see vt_test_expire_wait).
int launch_expire_wait(DeviceCtx* c, cudaStream_t s);
int launch_sgemm(DeviceCtx* c, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                 int variant, cudaStream_t s);
// Pipelined FFMA kernel (sgemm_ffma_sm100.cu); shape 0: 128 x 128 tiles, 1: 64 x 128, 2: 64 x 64.
bool sgemm_ffma_supported(const float* A, const float* B, const float* C, int64_t N, int64_t K);
double sgemm_ffma_plan(DeviceCtx* c, int shape, int64_t M, int64_t N, int64_t K, int forced, int* splits_out);
int launch_sgemm_ffma(DeviceCtx* c, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int shape,
                      cudaStream_t s);
double sgemm_tile_choice(DeviceCtx* c, const float* A, const float* B, const float* C, int64_t M, int64_t N, int64_t K,
                         int* variant);
int launch_sgemm_skinny(DeviceCtx* c, const float* A, const float* B, float* C, float* partials, int64_t M,
                        int64_t N, int64_t K, int ksplit, cudaStream_t s);
bool sgemm_tf32x3_supported(const float* A, const float* B, const float* C, int64_t M, int64_t N, int64_t K);
size_t sgemm_tf32x3_workspace_bytes(int64_t M, int64_t N, int64_t K);
int launch_sgemm_tf32x3(DeviceCtx* c, const float* A, const float* B, float* C, float* split, int64_t M, int64_t N,
                        int64_t K, cudaStream_t s, int parts = 3);
void sgemm_skinny_tma_plan(int64_t N, int64_t K, int sm_count, int* ctas, int* slabs, int* max_parts);
bool sgemm_skinny_tma_supported(const float* B, const float* C, int64_t M, int64_t N, int64_t K);
int launch_sgemm_skinny_tma(DeviceCtx* c, const float* A, const float* B, float* C, float* partials, int* tickets,
                            int64_t M, int64_t N, int64_t K, cudaStream_t s);
constexpr int SKINNY_UMMA_MAX_ROWS = 128;   // rows of A one launch of the row-panel tensor-core kernel takes
void sgemm_skinny_umma_plan(int64_t M, int64_t N, int64_t K, int sm_count, int* ctas, int* slabs, int* max_parts);
bool sgemm_skinny_umma_supported(const float* A, const float* B, const float* C, int64_t M, int64_t N, int64_t K);
int launch_sgemm_skinny_umma(DeviceCtx* c, const float* A, const float* B, float* C, float* partials, int* tickets,
                             int64_t M, int64_t N, int64_t K, cudaStream_t s);
void sgemm_tall_umma_plan(int64_t M, int64_t N, int64_t K, int sm_count, int* max_parts, size_t* b_and_lo_bytes);
bool sgemm_tall_umma_supported(const float* A, const float* B, const float* C, int64_t M, int64_t N, int64_t K);
int launch_sgemm_tall_umma(DeviceCtx* c, const float* A, const float* B, float* C, float* partials, int* tickets,
                           float* b_and_lo, int64_t M, int64_t N, int64_t K, int64_t ldb, int64_t ldc, cudaStream_t s);
size_t sgemm_skinny_partials_bytes(int64_t M, int64_t N, int64_t K, int sm_count, int* ksplit_out);
int launch_i8_tile_program(DeviceCtx* c, const int8_t* A, const int8_t* B, int32_t* C, int64_t lda, int64_t ldb,
                           int64_t ldc, int64_t n_tiles, const int64_t* d_c_off, const int64_t* d_term_begin,
                           const int64_t* d_a_off, const int64_t* d_b_off, cudaStream_t s);

}  // namespace vt
