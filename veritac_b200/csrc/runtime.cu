// Per-device contexts, error text, workspace and TMA tensor-map encoding.
#include "runtime.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>

#include "ptx_sm100.cuh"

namespace vt {

namespace {
constexpr int kMaxDevices = 16;
DeviceCtx g_ctx[kMaxDevices];
std::mutex g_mu;
std::atomic<long long> g_launches{0};
thread_local char t_err[512] = "";

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof(t_err), fmt, ap);
  va_end(ap);
  return code;
}

int fail_cuda(cudaError_t e, const char* what) {
  return fail(VT_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

const char* last_error_text() { return t_err; }
void clear_error_text() { t_err[0] = 0; }
long long launch_count() { return g_launches.load(); }
void count_launch(int n) { g_launches.fetch_add(n); }

DeviceCtx* ctx_for(int dev) {
  if (dev < 0 || dev >= kMaxDevices) {
    fail(VT_ERR_INVALID, "device ordinal %d out of range", dev);
    return nullptr;
  }
  cudaError_t e = cudaSetDevice(dev);
  if (e != cudaSuccess) {
    fail_cuda(e, "cudaSetDevice");
    return nullptr;
  }
  DeviceCtx* c = &g_ctx[dev];
  if (c->ready.load(std::memory_order_acquire)) return c;
  std::lock_guard<std::mutex> lock(g_mu);
  if (c->ready.load(std::memory_order_acquire)) return c;
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) {
    fail_cuda(e, "cudaGetDeviceProperties");
    return nullptr;
  }
  if (prop.major != 10) {
    fail(VT_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", dev, prop.major,
         prop.minor);
    return nullptr;
  }
  c->dev = dev;
  c->sm_count = prop.multiProcessorCount;
  c->smem_optin = prop.sharedMemPerBlockOptin;
#define CTX_TRY(expr)              \
  do {                             \
    e = (expr);                    \
    if (e != cudaSuccess) {        \
      fail_cuda(e, #expr);         \
      return nullptr;              \
    }                              \
  } while (0)
  CTX_TRY(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
  CTX_TRY(cudaStreamCreateWithFlags(&c->copy_in, cudaStreamNonBlocking));
  CTX_TRY(cudaStreamCreateWithFlags(&c->copy_out, cudaStreamNonBlocking));
  CTX_TRY(cudaMalloc(&c->status, sizeof(int)));
  CTX_TRY(cudaMemset(c->status, 0, sizeof(int)));
  CTX_TRY(cudaMallocHost(&c->status_host, sizeof(int)));
  CTX_TRY(cudaMalloc(&c->tickets, kTicketCount * sizeof(int)));
  CTX_TRY(cudaMemset(c->tickets, 0, kTicketCount * sizeof(int)));
  for (auto& ev : c->ev) CTX_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  CTX_TRY(cudaEventCreateWithFlags(&c->staging_consumed, cudaEventDisableTiming));
#undef CTX_TRY
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
      fail(VT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
      return nullptr;
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  c->ready.store(true, std::memory_order_release);
  return c;
}

void* ctx_workspace(DeviceCtx* c, int slot, size_t bytes) {
  if (bytes == 0) bytes = 256;
  if (c->ws_bytes[slot] >= bytes) return c->ws[slot];
  // Growing: nothing may still be using the old block.
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess && c->ws[slot]) e = cudaFree(c->ws[slot]);
  c->ws[slot] = nullptr;
  c->ws_bytes[slot] = 0;
  if (e == cudaSuccess) e = cudaMalloc(&c->ws[slot], bytes);
  if (e != cudaSuccess) {
    fail_cuda(e, "workspace cudaMalloc");
    return nullptr;
  }
  c->ws_bytes[slot] = bytes;
  return c->ws[slot];
}

void* ctx_pinned_staging(DeviceCtx* c, size_t bytes) {
  if (bytes == 0) bytes = 256;
  cudaError_t e = cudaEventSynchronize(c->staging_consumed);   // a never-recorded event is complete
  if (e == cudaSuccess && c->staging_bytes < bytes) {
    if (c->staging) e = cudaFreeHost(c->staging);
    c->staging = nullptr;
    c->staging_bytes = 0;
    if (e == cudaSuccess) e = cudaMallocHost(&c->staging, bytes);
    if (e == cudaSuccess) c->staging_bytes = bytes;
  }
  if (e != cudaSuccess) {
    fail_cuda(e, "pinned staging block");
    return nullptr;
  }
  return c->staging;
}

int ctx_check_status(DeviceCtx* c, cudaStream_t s) {
  VT_CUDA(cudaMemcpyAsync(c->status_host, c->status, sizeof(int), cudaMemcpyDeviceToHost, s));
  VT_CUDA(cudaStreamSynchronize(s));
  const int st = *c->status_host;
  if (st != KSTAT_OK) {
    VT_CUDA(cudaMemsetAsync(c->status, 0, sizeof(int), s));
    VT_CUDA(cudaMemsetAsync(c->tickets, 0, kTicketCount * sizeof(int), s));   // an aborted kernel may have left counts behind
    VT_CUDA(cudaStreamSynchronize(s));
    return fail(VT_ERR_DEVICE_WAIT, "a kernel gave up on a bounded device-side wait (status %d)", st);
  }
  return VT_OK;
}

void ctx_destroy_all() {
  std::lock_guard<std::mutex> lock(g_mu);
  for (int d = 0; d < kMaxDevices; ++d) {
    DeviceCtx* c = &g_ctx[d];
    if (!c->ready) continue;
    if (cudaSetDevice(d) != cudaSuccess) continue;
    cudaDeviceSynchronize();
    for (int i = 0; i < 4; ++i)
      if (c->ws[i]) cudaFree(c->ws[i]);
    if (c->status) cudaFree(c->status);
    if (c->status_host) cudaFreeHost(c->status_host);
    if (c->staging) cudaFreeHost(c->staging);
    if (c->staging_consumed) cudaEventDestroy(c->staging_consumed);
    if (c->tickets) cudaFree(c->tickets);
    for (auto& ev : c->ev)
      if (ev) cudaEventDestroy(ev);
    if (c->stream) cudaStreamDestroy(c->stream);
    if (c->copy_in) cudaStreamDestroy(c->copy_in);
    if (c->copy_out) cudaStreamDestroy(c->copy_out);
    c->ready.store(false, std::memory_order_release);
    c->~DeviceCtx();
    new (c) DeviceCtx();
  }
}

namespace {
// One warp waits for a barrier that expects an arrival nobody makes.  The wait is the production one
// (mbar_wait): it gives up after `limit` cycles, records its code in the abort word, and the kernel passes
// that on to the device status word exactly as the GEMM kernels do.
__global__ void __launch_bounds__(32) expire_wait_kernel(int* __restrict__ status, long long limit) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_word = 0;
    fence_mbar_init();
  }
  __syncwarp();
  const bool done = mbar_wait(&bar, 0, &abort_word, KSTAT_WAIT_EXPIRED_MMA, limit);
  __syncwarp();
  if (threadIdx.x == 0 && !done && abort_word != 0) atomicCAS(status, 0, abort_word);
}
}  // namespace

int launch_expire_wait(DeviceCtx* c, cudaStream_t s) {
  expire_wait_kernel<<<1, 32, 0, s>>>(c->status, c->wait_limit_cycles);
  count_launch();
  VT_CUDA(cudaGetLastError());
  return VT_OK;
}

int encode_tmap_2d(CUtensorMap* out, CUtensorMapDataType dtype, int elem_bytes, const void* base, uint64_t inner,
                   uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner, uint32_t box_outer,
                   CUtensorMapSwizzle swizzle) {
  if (!g_encode) return fail(VT_ERR_CUDA, "tensor-map encoder not initialised");
  if (reinterpret_cast<uintptr_t>(base) & 15) return fail(VT_ERR_INVALID, "TMA base address must be 16-byte aligned");
  if (row_pitch_bytes & 15) return fail(VT_ERR_INVALID, "TMA row pitch must be a multiple of 16 bytes");
  if (box_inner * uint32_t(elem_bytes) != 128 || box_outer == 0 || box_outer > 256)
    return fail(VT_ERR_INVALID, "TMA box must be 128 bytes wide and at most 256 rows");
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_pitch_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_encode(out, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(VT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (inner %llu outer %llu box %ux%u)", int(r),
                (unsigned long long)inner, (unsigned long long)outer, box_inner, box_outer);
  return VT_OK;
}

}  // namespace vt
