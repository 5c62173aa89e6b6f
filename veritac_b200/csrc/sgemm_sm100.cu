// fp32 GEMM C[M,N] = A[M,K] * B[K,N] (row-major, C overwritten): the matmul loop nest that the
// reference emits as OpenMP C (specializations/cpu_gemm/emit_c.py:83-155 generates the nest,
// specializations/cpu_gemm/runner.py:155-190 times it), executed on the FP32 pipe.
//
//   sgemm_tile_kernel<RM,RN>  register-tiled FFMA kernel.  256 threads as a 16x16 grid; each thread
//       owns (4*RM)x(4*RN) outputs as RM x RN blocks of 4x4 spaced 64 apart, so a CTA covers
//       (64*RM)x(64*RN).  K is consumed 16 at a time through two shared-memory buffers: global loads
//       for step t+1 are issued into registers before the FFMAs of step t and stored (A transposed
//       so the inner loop reads float4s along M) after them, one __syncthreads per step.
//       The 128x128 form is limited by instruction issue, so it uses the packed fma.rn.f32x2 (two
//       rows of one column per instruction: the row pair comes straight from the float4 of A, the
//       column value is copied into both halves of a register pair), brings B in by cp.async (no
//       staging registers, which is what lets the packed form fit 128 registers without spills) and
//       lays a warp out as 4 x 8 threads.
//   sgemm_small_kernel        products too small to fill the GPU with 64x64 tiles: 32x32 CTA tile, K in
//       bursts of 256 split four ways inside the CTA (described at the kernel).
//   sgemm_skinny_kernel       M <= 16 ("decode-like") in true fp32: B is streamed exactly once.  A CTA owns
//       128 columns and a K range; B rows arrive through a 4-stage cp.async ring, its 4 warps take
//       8-row slices of each 32-row stage, keep 16x4 accumulators per thread, and fold through shared memory.  With a K split the
//       per-split partial tiles go to scratch memory and a second kernel sums them in split order
//       (deterministic, no atomics).
#include <atomic>
#include <mutex>

#include "ptx_sm100.cuh"
#include "runtime.h"

namespace vt {
namespace {

constexpr int SG_THREADS = 256;
constexpr int SG_BK = 16;

__device__ __forceinline__ void cp_async_16_zfill(float* smem_dst, const float* gmem_src, bool valid) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  const int bytes = valid ? 16 : 0;   // 0 source bytes => the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

// K split over CTAs ("splits" CTAs per output tile, each with its own range of K): every CTA leaves its partial
// tile in scratch memory (float4 slot `j` of thread `tid` at [(tile * splits + split) * kSlots + j] * kThreads + tid)
// and takes a ticket for the tile; the CTA that draws the last ticket adds the partial tiles in split order, its
// own included, so the sum does not depend on which CTA that is.  Nobody waits for anybody.
// Called by the kThreads threads (named barrier kBar) that have stored a partial tile; true in the last CTA.
template <int kThreads, int kBar>
__device__ __forceinline__ bool splitk_arrive(int tile, int splits, int* __restrict__ tickets, int* last_flag, int tid) {
  __threadfence();
  asm volatile("bar.sync %0, %1;" ::"n"(kBar), "n"(kThreads) : "memory");
  if (tid == 0) {
    const int arrived = atomicAdd(&tickets[tile], 1);
    const int last = arrived == splits - 1;
    if (last) tickets[tile] = 0;      // every CTA of the tile has arrived: the counter is free for the next launch
    *last_flag = last;
  }
  asm volatile("bar.sync %0, %1;" ::"n"(kBar), "n"(kThreads) : "memory");
  if (!*last_flag) return false;
  __threadfence();
  return true;
}
__device__ __forceinline__ float4 splitk_sum(const float4* __restrict__ first, size_t split_stride, int splits) {
  float4 sum = __ldcg(first);
#pragma unroll 4
  for (int s = 1; s < splits; ++s) {
    const float4 v = __ldcg(first + size_t(s) * split_stride);
    sum.x += v.x;
    sum.y += v.y;
    sum.z += v.z;
    sum.w += v.w;
  }
  return sum;
}


template <int RM, int RN, bool kGuard>
__global__ void __launch_bounds__(SG_THREADS, (RM * RN >= 4) ? 2 : 3)
sgemm_tile_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N,
                  int K, int tiles_m, int tiles_n, int group) {
  constexpr int BM = 64 * RM, BN = 64 * RN;
  constexpr int LDA = BM + 4;
  __shared__ __align__(16) float As[2][SG_BK][LDA];
  __shared__ __align__(16) float Bs[2][SG_BK][BN];

  // Grouped tile order: sweep all tile-columns for `group` tile-rows at a time (L2 reuse of B).
  int tm, tn;
  {
    const int t = blockIdx.x;
    const int per = group * tiles_n;
    const int g = t / per;
    const int w = t - g * per;
    const int rows = min(group, tiles_m - g * group);
    tn = w / rows;
    tm = g * group + (w - tn * rows);
  }
  const int m0 = tm * BM, n0 = tn * BN;
  const int tid = threadIdx.x;
  // Packed form: a warp is 4 (M) x 8 (N) threads and the 8 warps are 4 (M) x 2 (N), so that per K step a warp
  // reads 4 distinct float4s of A and 8 of B instead of 2 and 16.
  constexpr bool kPacked = RM * RN >= 4;
  const int tx = kPacked ? ((tid >> 5) & 1) * 8 + (tid & 7) : tid & 15;
  const int ty = kPacked ? (tid >> 6) * 4 + ((tid >> 3) & 3) : tid >> 4;
  constexpr bool kAsyncB = kPacked && !kGuard;

  const int a_row = tid >> 2;        // 0..63 (+64 per pass)
  const int a_k = (tid & 3) * 4;     // 0,4,8,12
  constexpr int B_F4_PER_ROW = 16 * RN;
  constexpr int B_ROWS_PER_PASS = SG_THREADS / B_F4_PER_ROW;  // 16 / RN
  const int b_k = tid / B_F4_PER_ROW;
  const int b_n = (tid % B_F4_PER_ROW) * 4;

  float4 pa[RM], pb[RN];
  // Running pointers for the unguarded path (advanced once per K step).
  const float* a_ptr = A + size_t(m0 + a_row) * K + a_k;
  const float* b_ptr = B + size_t(b_k) * N + n0 + b_n;
  const size_t a_pass = size_t(64) * K, b_pass = size_t(B_ROWS_PER_PASS) * N;

  auto load_tile = [&](int k0, int nbuf) {
#pragma unroll
    for (int i = 0; i < RM; ++i) {
      const int row = m0 + a_row + 64 * i;
      const int k = k0 + a_k;
      if constexpr (!kGuard) {
        pa[i] = __ldg(reinterpret_cast<const float4*>(a_ptr + i * a_pass));
      } else {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = (row < M && k + j < K) ? A[size_t(row) * K + k + j] : 0.f;
        pa[i] = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
#pragma unroll
    for (int i = 0; i < RN; ++i) {
      const int k = k0 + b_k + B_ROWS_PER_PASS * i;
      const int col = n0 + b_n;
      if constexpr (kAsyncB) {
        cp_async_16_zfill(&Bs[nbuf][b_k + B_ROWS_PER_PASS * i][b_n], b_ptr + i * b_pass, true);
      } else if constexpr (!kGuard) {
        pb[i] = __ldg(reinterpret_cast<const float4*>(b_ptr + i * b_pass));
      } else {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = (k < K && col + j < N) ? B[size_t(k) * N + col + j] : 0.f;
        pb[i] = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
    if constexpr (!kGuard) {
      a_ptr += SG_BK;
      b_ptr += size_t(SG_BK) * N;
    }
  };
  auto store_tile = [&](int buf) {
#pragma unroll
    for (int i = 0; i < RM; ++i) {
      const int r = a_row + 64 * i;
      As[buf][a_k + 0][r] = pa[i].x;
      As[buf][a_k + 1][r] = pa[i].y;
      As[buf][a_k + 2][r] = pa[i].z;
      As[buf][a_k + 3][r] = pa[i].w;
    }
    if constexpr (kAsyncB) {
      cp_async_commit();
      cp_async_wait<0>();             // this thread's part of B has landed; the barrier publishes it
    } else {
#pragma unroll
      for (int i = 0; i < RN; ++i)
        *reinterpret_cast<float4*>(&Bs[buf][b_k + B_ROWS_PER_PASS * i][b_n]) = pb[i];
    }
  };

  // acc[p][j] = rows (2p, 2p+1) of column j of this thread's (4*RM) x (4*RN) outputs.
  float2 acc[2 * RM][4 * RN];
#pragma unroll
  for (int p = 0; p < 2 * RM; ++p)
#pragma unroll
    for (int j = 0; j < 4 * RN; ++j) acc[p][j] = make_float2(0.f, 0.f);

  // Launched for overlap with the kernel before it on the stream (launch_overlapped): its blocks may be placed
  // while that kernel's last blocks run; nothing is read or written before it has completed.
  grid_dependency_wait();
  grid_launch_dependents();
  const int ktiles = (K + SG_BK - 1) / SG_BK;
  load_tile(0, 0);
  store_tile(0);
  __syncthreads();

  for (int kt = 0; kt < ktiles; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < ktiles) load_tile((kt + 1) * SG_BK, buf ^ 1);
#pragma unroll(kPacked ? 8 : SG_BK)
    for (int k = 0; k < SG_BK; ++k) {
      float a[4 * RM], b[4 * RN];
#pragma unroll
      for (int i = 0; i < RM; ++i) {
        const float4 v = *reinterpret_cast<const float4*>(&As[buf][k][64 * i + ty * 4]);
        a[4 * i + 0] = v.x; a[4 * i + 1] = v.y; a[4 * i + 2] = v.z; a[4 * i + 3] = v.w;
      }
#pragma unroll
      for (int j = 0; j < RN; ++j) {
        const float4 v = *reinterpret_cast<const float4*>(&Bs[buf][k][64 * j + tx * 4]);
        b[4 * j + 0] = v.x; b[4 * j + 1] = v.y; b[4 * j + 2] = v.z; b[4 * j + 3] = v.w;
      }
      if constexpr (kPacked) {
#pragma unroll
        for (int j = 0; j < 4 * RN; ++j) {
          const float2 bb = make_float2(b[j], b[j]);
#pragma unroll
          for (int p = 0; p < 2 * RM; ++p) acc[p][j] = __ffma2_rn(make_float2(a[2 * p], a[2 * p + 1]), bb, acc[p][j]);
        }
      } else {
#pragma unroll
        for (int p = 0; p < 2 * RM; ++p)
#pragma unroll
          for (int j = 0; j < 4 * RN; ++j) {
            acc[p][j].x = fmaf(a[2 * p], b[j], acc[p][j].x);
            acc[p][j].y = fmaf(a[2 * p + 1], b[j], acc[p][j].y);
          }
      }
    }
    if (kt + 1 < ktiles) store_tile(buf ^ 1);
    __syncthreads();
  }

  auto cell = [&](int i, int j) { return (i & 1) ? acc[i >> 1][j].y : acc[i >> 1][j].x; };
#pragma unroll
  for (int i = 0; i < 4 * RM; ++i) {
    const int row = m0 + 64 * (i >> 2) + ty * 4 + (i & 3);
#pragma unroll
    for (int j = 0; j < RN; ++j) {
      const int col = n0 + 64 * j + tx * 4;
      if constexpr (!kGuard) {
        *reinterpret_cast<float4*>(C + size_t(row) * N + col) =
            make_float4(cell(i, 4 * j), cell(i, 4 * j + 1), cell(i, 4 * j + 2), cell(i, 4 * j + 3));
      } else {
        if (row < M) {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (col + e < N) C[size_t(row) * N + col + e] = cell(i, 4 * j + e);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Skinny: M <= 16, N % 4 == 0.  grid = (N/128 rounded up, ksplit), 128 threads.
// B rows stream through a 4-stage cp.async ring (32 rows x 128 columns = 16 KiB per stage, three
// CTAs per SM => ~150 KiB of B in flight per SM); the matching 32 x 16 slice of A goes through
// registers one stage ahead and lands transposed ([k][m]) so the inner loop reads it as broadcast
// float4s.  Each of the 4 warps takes 8 of a stage's 32 rows for all 128 columns (lane = 4 columns)
// and keeps a 16 x 4 accumulator per thread; warps fold in a fixed order at the end.
// ---------------------------------------------------------------------------------------------
constexpr int SK_M = 16;
constexpr int SK_COLS = 128;
constexpr int SK_WARPS = 4;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_KC = 32;                      // K rows per stage
constexpr int SK_RW = SK_KC / SK_WARPS;        // rows of a stage each warp consumes
constexpr int SK_STAGES = 4;
constexpr int SK_B_STAGE = SK_KC * SK_COLS;    // floats
constexpr int SK_A_STAGE = SK_KC * SK_M;       // floats
constexpr size_t SK_SMEM_BYTES = size_t(SK_STAGES) * (SK_B_STAGE + SK_A_STAGE) * sizeof(float);

__global__ void __launch_bounds__(SK_THREADS, 3)
sgemm_skinny_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ out, int M, int N,
                    int K, int k_per_split) {
  extern __shared__ __align__(16) float sk_smem[];
  float* Bs = sk_smem;                                   // [stage][32][128]
  float* As = sk_smem + SK_STAGES * SK_B_STAGE;          // [stage][32][16]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * SK_COLS;
  const int kbeg = blockIdx.y * k_per_split;
  const int kend = min(K, kbeg + k_per_split);
  const int nchunks = kend > kbeg ? (kend - kbeg + SK_KC - 1) / SK_KC : 0;

  const int a_m = tid >> 3, a_k = (tid & 7) * 4;         // this thread's 4 elements of a stage's A slice

  auto issue_b = [&](int chunk) {                        // 8 x 16-byte copies per thread
    float* dst = Bs + (chunk % SK_STAGES) * SK_B_STAGE;
    const int k0 = kbeg + chunk * SK_KC;
#pragma unroll
    for (int i = 0; i < SK_KC * SK_COLS / 4 / SK_THREADS; ++i) {
      const int idx = tid + SK_THREADS * i;
      const int row = idx >> 5, c4 = (idx & 31) * 4;
      const bool ok = (k0 + row < kend) && (n0 + c4 < N);
      const float* src = ok ? B + size_t(k0 + row) * N + n0 + c4 : B;
      cp_async_16_zfill(dst + row * SK_COLS + c4, src, ok);
    }
  };
  auto load_a = [&](int chunk, float (&v)[4]) {
    const int k0 = kbeg + chunk * SK_KC + a_k;
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = (a_m < M && k0 + j < kend) ? __ldg(A + size_t(a_m) * K + k0 + j) : 0.f;
  };
  auto store_a = [&](int chunk, const float (&v)[4]) {
    float* dst = As + (chunk % SK_STAGES) * SK_A_STAGE;
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[(a_k + j) * SK_M + a_m] = v[j];
  };

  float2 acc[SK_M / 2][4];   // acc[p][c] = rows (2p, 2p+1) of column c: one fma.rn.f32x2 updates both
#pragma unroll
  for (int m = 0; m < SK_M / 2; ++m)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[m][j] = make_float2(0.f, 0.f);

  // Prologue: stages 0 .. SK_STAGES-2 (one commit per stage, empty ones included, so the
  // wait below always counts the same number of groups).
  for (int c = 0; c < SK_STAGES - 1; ++c) {
    if (c < nchunks) {
      issue_b(c);
      float v[4];
      load_a(c, v);
      store_a(c, v);
    }
    cp_async_commit();
  }

  for (int it = 0; it < nchunks; ++it) {
    cp_async_wait<SK_STAGES - 2>();   // chunk `it` has landed (for this thread's copies)
    __syncthreads();                  // ... and for everyone's; everyone is also done with chunk it-1
    const int nxt = it + SK_STAGES - 1;
    float av[4];
    const bool more = nxt < nchunks;
    if (more) {
      issue_b(nxt);
      load_a(nxt, av);
    }
    cp_async_commit();

    const float* bs = Bs + (it % SK_STAGES) * SK_B_STAGE + (warp * SK_RW) * SK_COLS + lane * 4;
    const float* as = As + (it % SK_STAGES) * SK_A_STAGE + (warp * SK_RW) * SK_M;
#pragma unroll
    for (int r = 0; r < SK_RW; ++r) {
      const float4 b = *reinterpret_cast<const float4*>(bs + r * SK_COLS);
      const float2 bx = make_float2(b.x, b.x), by = make_float2(b.y, b.y), bz = make_float2(b.z, b.z),
                   bw = make_float2(b.w, b.w);
#pragma unroll
      for (int mq = 0; mq < SK_M / 4; ++mq) {
        const float4 a4 = *reinterpret_cast<const float4*>(as + r * SK_M + 4 * mq);
        const float2 a01 = make_float2(a4.x, a4.y), a23 = make_float2(a4.z, a4.w);
        acc[2 * mq][0] = __ffma2_rn(a01, bx, acc[2 * mq][0]);
        acc[2 * mq][1] = __ffma2_rn(a01, by, acc[2 * mq][1]);
        acc[2 * mq][2] = __ffma2_rn(a01, bz, acc[2 * mq][2]);
        acc[2 * mq][3] = __ffma2_rn(a01, bw, acc[2 * mq][3]);
        acc[2 * mq + 1][0] = __ffma2_rn(a23, bx, acc[2 * mq + 1][0]);
        acc[2 * mq + 1][1] = __ffma2_rn(a23, by, acc[2 * mq + 1][1]);
        acc[2 * mq + 1][2] = __ffma2_rn(a23, bz, acc[2 * mq + 1][2]);
        acc[2 * mq + 1][3] = __ffma2_rn(a23, bw, acc[2 * mq + 1][3]);
      }
    }
    if (more) store_a(nxt, av);       // read after a later __syncthreads
  }
  cp_async_wait<0>();

  // Fold the warps' partial tiles in warp order (fixed order => reproducible bits); the ring's
  // first stage is free by now and serves as the 16 x 128 fold buffer.
  float* red = Bs;
  for (int w = 0; w < SK_WARPS; ++w) {
    __syncthreads();
    if (warp == w) {
#pragma unroll
      for (int m = 0; m < SK_M; ++m) {
        float4* p = reinterpret_cast<float4*>(red + m * SK_COLS + lane * 4);
        float4 v = (w == 0) ? make_float4(0.f, 0.f, 0.f, 0.f) : *p;
        const float2 c0 = acc[m >> 1][0], c1 = acc[m >> 1][1], c2 = acc[m >> 1][2], c3 = acc[m >> 1][3];
        v.x += (m & 1) ? c0.y : c0.x; v.y += (m & 1) ? c1.y : c1.x;
        v.z += (m & 1) ? c2.y : c2.x; v.w += (m & 1) ? c3.y : c3.x;
        *p = v;
      }
    }
  }
  __syncthreads();
  // out is C itself (no K split) or the partial tile of this split: [split][M][N].
  float* dst = out + size_t(blockIdx.y) * size_t(M) * size_t(N);
  for (int i = tid; i < SK_M * (SK_COLS / 4); i += SK_THREADS) {
    const int m = i / (SK_COLS / 4), c4 = i - m * (SK_COLS / 4);
    const int col = n0 + c4 * 4;
    if (m < M && col < N)
      *reinterpret_cast<float4*>(dst + size_t(m) * N + col) = *reinterpret_cast<const float4*>(red + m * SK_COLS + c4 * 4);
  }
}

__global__ void __launch_bounds__(256)
sgemm_skinny_reduce_kernel(const float* __restrict__ partials, float* __restrict__ C, int64_t mn4, int ksplit) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= mn4) return;
  const float4* p = reinterpret_cast<const float4*>(partials);
  float4 s = p[i];
  for (int k = 1; k < ksplit; ++k) {
    const float4 v = p[int64_t(k) * mn4 + i];
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  reinterpret_cast<float4*>(C)[i] = s;
}

// ---------------------------------------------------------------------------------------------
// Small products (the reference's own 256^3 demo): a grid of 64x64 tiles cannot fill 148 SMs and a
// CTA that walks K in 16 dependent load-compute steps pays the global-load latency 16 times.
// Here a CTA owns a 32x32 tile, brings 256 values of K for it into shared memory in one burst of
// cp.async (A as 32 rows of K, B as 256 rows of 32), and its 256 threads work as four groups that
// each take a quarter of those K values for the whole tile (4x4 outputs per thread, operands read
// as float4: A along K, B along N).  The four partial tiles are added in group order through
// shared memory.  True fp32 arithmetic.  Needs K % 4 == 0, N % 4 == 0 and 16-byte aligned operands
// (cp.async moves 16 bytes); M, N, K are otherwise free (edges are zero-filled).
// ---------------------------------------------------------------------------------------------
constexpr int SS_TILE = 32;
constexpr int SS_KC = 256;                        // values of K per burst
constexpr int SS_APITCH = SS_KC + 4;              // floats; keeps the four rows a warp reads in different banks
constexpr int SS_THREADS = 256;
constexpr size_t SS_SMEM_BYTES = size_t(SS_TILE * SS_APITCH + SS_KC * SS_TILE) * sizeof(float);

__global__ void __launch_bounds__(SS_THREADS, 2)
sgemm_small_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N,
                   int K, int tiles_n, int n_tiles, int splits, int k_per_split, float* __restrict__ partials,
                   int* __restrict__ tickets) {
  extern __shared__ __align__(16) float ss_smem[];
  float* As = ss_smem;                            // [32][SS_APITCH]
  float* Bs = ss_smem + SS_TILE * SS_APITCH;      // [256][32]
  const int tid = threadIdx.x;
  const int split = blockIdx.x / n_tiles, tile = blockIdx.x - split * n_tiles;   // K split: as in sgemm_tile_kernel
  const int m0 = (tile / tiles_n) * SS_TILE, n0 = (tile % tiles_n) * SS_TILE;
  const int k_begin = split * k_per_split;
  const int k_end = min(K, k_begin + k_per_split);
  const int kg = tid >> 6;                        // which quarter of a burst's K values
  const int t = tid & 63, tx = t & 7, ty = t >> 3;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // This kernel is a few microseconds long, about as long as the gap between two launches: it is launched so
  // that its CTAs may be placed while the kernel before it on the stream is still running, and waits here,
  // before its first access to global memory, for that kernel to complete.
  grid_dependency_wait();
  grid_launch_dependents();

  for (int k0 = k_begin; k0 < k_end; k0 += SS_KC) {
    if (k0 > k_begin) __syncthreads();            // everyone is done with the previous burst
    // A: 32 rows x 64 float4; B: 256 rows x 8 float4.  2048 copies each, 8 + 8 per thread.
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = tid + SS_THREADS * i;
      const int row = idx >> 6, c4 = (idx & 63) * 4;
      const bool ok = (m0 + row < M) && (k0 + c4 < k_end);
      cp_async_16_zfill(As + row * SS_APITCH + c4, ok ? A + size_t(m0 + row) * K + k0 + c4 : A, ok);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = tid + SS_THREADS * i;
      const int row = idx >> 3, c4 = (idx & 7) * 4;
      const bool ok = (k0 + row < k_end) && (n0 + c4 < N);
      cp_async_16_zfill(Bs + row * SS_TILE + c4, ok ? B + size_t(k0 + row) * N + n0 + c4 : B, ok);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    const float* a_base = As + (ty * 4) * SS_APITCH + kg * (SS_KC / 4);
    const float* b_base = Bs + (kg * (SS_KC / 4)) * SS_TILE + tx * 4;
#pragma unroll 4
    for (int k = 0; k < SS_KC / 4; k += 4) {
      float4 a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const float4*>(a_base + i * SS_APITCH + k);
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = *reinterpret_cast<const float4*>(b_base + (k + j) * SS_TILE);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[i][0] = fmaf(a[i].x, b[0].x, acc[i][0]);
        acc[i][1] = fmaf(a[i].x, b[0].y, acc[i][1]);
        acc[i][2] = fmaf(a[i].x, b[0].z, acc[i][2]);
        acc[i][3] = fmaf(a[i].x, b[0].w, acc[i][3]);
        acc[i][0] = fmaf(a[i].y, b[1].x, acc[i][0]);
        acc[i][1] = fmaf(a[i].y, b[1].y, acc[i][1]);
        acc[i][2] = fmaf(a[i].y, b[1].z, acc[i][2]);
        acc[i][3] = fmaf(a[i].y, b[1].w, acc[i][3]);
        acc[i][0] = fmaf(a[i].z, b[2].x, acc[i][0]);
        acc[i][1] = fmaf(a[i].z, b[2].y, acc[i][1]);
        acc[i][2] = fmaf(a[i].z, b[2].z, acc[i][2]);
        acc[i][3] = fmaf(a[i].z, b[2].w, acc[i][3]);
        acc[i][0] = fmaf(a[i].w, b[3].x, acc[i][0]);
        acc[i][1] = fmaf(a[i].w, b[3].y, acc[i][1]);
        acc[i][2] = fmaf(a[i].w, b[3].z, acc[i][2]);
        acc[i][3] = fmaf(a[i].w, b[3].w, acc[i][3]);
      }
    }
  }

  // Groups 1..3 leave their partial tiles in shared memory; group 0 adds them in group order.
  __syncthreads();
  float* red = ss_smem;                           // [3][64 threads][16], written as float4s
  if (kg > 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      *reinterpret_cast<float4*>(red + ((kg - 1) * 64 + t) * 16 + i * 4) =
          make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
  }
  __syncthreads();
  if (kg == 0) {
#pragma unroll
    for (int g = 0; g < 3; ++g)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 v = *reinterpret_cast<const float4*>(red + (g * 64 + t) * 16 + i * 4);
        acc[i][0] += v.x;
        acc[i][1] += v.y;
        acc[i][2] += v.z;
        acc[i][3] += v.w;
      }
    const int col = n0 + tx * 4;
    if (splits == 1) {
      if (col < N) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = m0 + ty * 4 + i;
          if (row < M)
            *reinterpret_cast<float4*>(C + size_t(row) * N + col) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        }
      }
      return;
    }
    constexpr size_t kSplitStride = 4 * 64;          // float4s per partial tile
    float4* first = reinterpret_cast<float4*>(partials) + size_t(tile) * splits * kSplitStride + t;
    float4* mine = first + size_t(split) * kSplitStride;
#pragma unroll
    for (int i = 0; i < 4; ++i) __stcg(mine + i * 64, make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]));
    int* last_flag = reinterpret_cast<int*>(ss_smem + 3 * 64 * 16);   // behind the fold area above
    if (!splitk_arrive<64, 1>(tile, splits, tickets, last_flag, t)) return;
    if (col < N) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = m0 + ty * 4 + i;
        if (row < M) *reinterpret_cast<float4*>(C + size_t(row) * N + col) = splitk_sum(first + i * 64, kSplitStride, splits);
      }
    }
  }
}

bool sgemm_small_ok(const float* A, const float* B, const float* C, int64_t N, int64_t K) {
  return N % 4 == 0 && K % 4 == 0 &&
         ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) == 0;
}

// How many CTAs share the K range of one output tile.  A grid that fills at most half the CTA slots of the GPU
// (`slots`) leaves SMs idle, or one CTA alone on an SM with nothing to overlap its loads; splitting K fills one
// wave instead.  Every split gets at least `min_k` values of K and a tile at most `most` partial tiles.
// `forced` (vt_test_set_sgemm_splits) overrides the count.
constexpr int kMaxSplits = 16;
int splits_for(long long tiles, int K, int slots, int min_k, int most, int forced) {
  long long s = 1;
  if (forced != 0) s = forced < 0 ? -forced : forced;
  else if (tiles * 2 <= slots) s = slots / tiles;
  if (s > most) s = most;
  if (s > K / min_k) s = K / min_k;
  if (tiles > kTicketCount) s = 1;     // one arrival counter per tile
  return s < 1 ? 1 : int(s);
}
// K values per split (a multiple of `step`) and the number of splits that then have any.
void split_ranges(int K, int step, int* splits, int* k_per_split) {
  const int steps = (K + step - 1) / step;
  const int per = (steps + *splits - 1) / *splits;
  *k_per_split = per * step;
  *splits = (steps + per - 1) / per;
}

int launch_small(DeviceCtx* c, const float* A, const float* B, float* C, int M, int N, int K, cudaStream_t s) {
  if (!sgemm_small_ok(A, B, C, N, K))
    return fail(VT_ERR_UNSUPPORTED, "the 32x32-tile kernel needs N %% 4 == 0, K %% 4 == 0 and 16-byte aligned operands");
  const int tiles_m = (M + SS_TILE - 1) / SS_TILE, tiles_n = (N + SS_TILE - 1) / SS_TILE;
  const long long tiles = 1LL * tiles_m * tiles_n;
  if (tiles > 0x7fffffffLL) return fail(VT_ERR_INVALID, "sgemm tile count overflows int");
  int splits = splits_for(tiles, K, 2 * c->sm_count, 2 * SS_KC, kMaxSplits, c->sgemm_force_splits), k_per_split;
  split_ranges(K, SS_KC, &splits, &k_per_split);
  float* partials = nullptr;
  if (splits > 1) {
    partials = static_cast<float*>(ctx_workspace(c, 3, size_t(tiles) * splits * SS_TILE * SS_TILE * sizeof(float)));
    if (!partials) return VT_ERR_CUDA;
  }
  constexpr uint32_t kAttrBit = 1u << 3;       // once per device: this launch is a few microseconds long
  if (!(c->func_attr_mask & kAttrBit)) {
    VT_CUDA(cudaFuncSetAttribute(sgemm_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SS_SMEM_BYTES)));
    c->func_attr_mask |= kAttrBit;
  }
  VT_CUDA(launch_overlapped(sgemm_small_kernel, unsigned(tiles * splits), unsigned(SS_THREADS), size_t(SS_SMEM_BYTES), s, A,
                            B, C, M, N, K, tiles_n, int(tiles), splits, k_per_split, partials, c->tickets));
  count_launch();
  VT_CUDA(cudaGetLastError());
  return VT_OK;
}

template <int RM, int RN>
int launch_tile(const float* A, const float* B, float* C, int M, int N, int K, cudaStream_t s) {
  constexpr int BM = 64 * RM, BN = 64 * RN;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const long long tiles = 1LL * tiles_m * tiles_n;
  if (tiles > 0x7fffffffLL) return fail(VT_ERR_INVALID, "sgemm tile count overflows int");
  const int group = tiles_m < 8 ? tiles_m : 8;
  const bool aligned =
      ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) == 0;
  const bool full = aligned && M % BM == 0 && N % BN == 0 && K % SG_BK == 0;
  if (full)
    VT_CUDA(launch_overlapped(sgemm_tile_kernel<RM, RN, false>, unsigned(tiles), unsigned(SG_THREADS), size_t(0), s, A, B,
                              C, M, N, K, tiles_m, tiles_n, group));
  else
    VT_CUDA(launch_overlapped(sgemm_tile_kernel<RM, RN, true>, unsigned(tiles), unsigned(SG_THREADS), size_t(0), s, A, B,
                              C, M, N, K, tiles_m, tiles_n, group));
  count_launch();
  VT_CUDA(cudaGetLastError());
  return VT_OK;
}

}  // namespace

size_t sgemm_skinny_partials_bytes(int64_t M, int64_t N, int64_t K, int sm_count, int* ksplit_out) {
  // Three CTAs are resident per SM.  The K split is the one that minimises a simple cost model:
  // whole "waves" of resident CTAs (a last wave that is mostly empty costs as much as a full one)
  // times the extra traffic of writing and re-reading ksplit partial tiles.  A split is never
  // shorter than 8 stages of SK_KC rows, and splits have (nearly) equal stage counts.
  const int64_t col_ctas = (N + SK_COLS - 1) / SK_COLS;
  const int64_t chunks = (K + SK_KC - 1) / SK_KC;
  const int64_t max_split = chunks / 8 > 0 ? (chunks / 8 < 64 ? chunks / 8 : 64) : 1;
  const double slots = 3.0 * sm_count;
  int64_t best = 1;
  double best_cost = 1e300;
  for (int64_t cand = 1; cand <= max_split; ++cand) {
    const int64_t per = (chunks + cand - 1) / cand;
    const int64_t ks = (chunks + per - 1) / per;          // the split count this stage count really gives
    const double waves = double(col_ctas * ks) / slots;
    const double rounds = waves <= 1.0 ? 1.0 : double(int64_t(waves + 0.999999));
    // fewer CTAs than slots: the idle SMs' share of bandwidth is not lost, but parallelism is
    const double fill = waves < 1.0 ? waves : waves / rounds;
    const double extra = ks > 1 ? 1.0 + double(ks) * 2.0 * double(M) / double(K) : 1.0;
    const double cost = extra / (0.15 + 0.85 * fill);
    if (cost < best_cost - 1e-12) {
      best_cost = cost;
      best = ks;
    }
  }
  if (ksplit_out) *ksplit_out = int(best);
  return best > 1 ? size_t(best) * size_t(M) * size_t(N) * sizeof(float) : 0;
}

int launch_sgemm_skinny(DeviceCtx* c, const float* A, const float* B, float* C, float* partials, int64_t M,
                        int64_t N, int64_t K, int ksplit, cudaStream_t s) {
  (void)c;
  if (M > SK_M || N % 4 != 0) return fail(VT_ERR_UNSUPPORTED, "skinny kernel needs M <= 16 and N %% 4 == 0");
  if ((reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) | reinterpret_cast<uintptr_t>(partials)) & 15)
    return fail(VT_ERR_INVALID, "skinny kernel operands must be 16-byte aligned");
  if (ksplit < 1) ksplit = 1;
  if (ksplit > 1 && !partials) return fail(VT_ERR_INVALID, "K split needs a partials buffer");
  const int64_t chunks = (K + SK_KC - 1) / SK_KC;
  const int k_per_split = int((chunks + ksplit - 1) / ksplit) * SK_KC;
  dim3 grid(unsigned((N + SK_COLS - 1) / SK_COLS), unsigned(ksplit));
  float* out = ksplit > 1 ? partials : C;
  // Opt in to 72 KiB of dynamic shared memory (a per-device function attribute; setting it again is harmless).
  VT_CUDA(cudaFuncSetAttribute(sgemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SK_SMEM_BYTES)));
  sgemm_skinny_kernel<<<grid, SK_THREADS, SK_SMEM_BYTES, s>>>(A, B, out, int(M), int(N), int(K), k_per_split);
  count_launch();
  if (ksplit > 1) {
    const int64_t mn4 = M * N / 4;
    sgemm_skinny_reduce_kernel<<<unsigned((mn4 + 255) / 256), 256, 0, s>>>(partials, C, mn4, ksplit);
    count_launch();
  }
  VT_CUDA(cudaGetLastError());
  return VT_OK;
}

// Which FFMA kernel to run, and about how long it will take (seconds).  First design (sgemm_tile_kernel,
// sgemm_small_kernel): the work of the padded tile grid over the rate that tile shape reaches (measured: 58, 32 and
// 32 TFLOPS for 128-, 64- and 32-wide tiles with every SM busy), scaled down while the grid has fewer CTAs than
// SMs; the smallest tile has to win by 10 %; the 32-wide kernel splits K over several CTAs per tile when its grid is
// small (launch_small), which adds about 4 us.  Measured points the rule reproduces: 256^3 6.6 (32-wide) against
// 12.3 us (64-wide), 512^3 13.3 against 20.5 us, 8192 x 16 x 8192 151 against 399 us, 65536 x 16 x 1024 140 against
// 281 us, 8192 x 256 x 8192 0.91 ms (128-wide) against 1.07 ms, 256 x 256 x 8192 42 us (32-wide, split four ways).
// Second design (sgemm_ffma_kernel): sgemm_ffma_plan's model, which includes its cluster K split; it takes the
// mid-sized products (640^3: 18 us against 24).
double sgemm_tile_choice(DeviceCtx* c, const float* A, const float* B, const float* C, int64_t M, int64_t N, int64_t K,
                         int* variant) {
  const int sm_count = c->sm_count;
  const bool small_ok = sgemm_small_ok(A, B, C, N, K);
  static const double kRate[3] = {58e12, 32e12, 32e12};
  static const double kBias[3] = {1.0, 1.0, 1.1};
  static const int kTile[3] = {128, 64, 32};
  static const int kVariant[3] = {VT_SGEMM_TILE128, VT_SGEMM_TILE64, VT_SGEMM_TILE32};
  double best = 0;
  *variant = VT_SGEMM_TILE64;
  for (int i = 0; i < 3; ++i) {
    if (i == 2 && !small_ok) continue;
    const double tm = double((M + kTile[i] - 1) / kTile[i]), tn = double((N + kTile[i] - 1) / kTile[i]);
    const double work = 2.0 * tm * tn * kTile[i] * kTile[i] * double(K);
    int splits = 1, per = int(K);
    if (i == 2 && tm * tn < 1e9) {
      splits = splits_for((long long)(tm * tn), int(K), 2 * sm_count, 2 * SS_KC, kMaxSplits, 0);
      split_ranges(int(K), SS_KC, &splits, &per);
      if (per > K) per = int(K);
    }
    const double ctas = tm * tn * splits;
    const double busy = ctas < sm_count ? ctas / sm_count : 1.0;
    double t = 5.0e-6 + work / (kRate[i] * busy) * kBias[i];      // 5 us: what a launch costs beside its loop
    if (i == 2) {
      // The 32-wide kernel does not overlap a burst's loads with its arithmetic, so what counts is how many bursts
      // the busiest SM works through: one CTA alone on an SM takes 2.67 us per burst of 256 values of K, two CTAs
      // sharing an SM 4.36 us for a burst each (measured; 212 x 716 x 2828 is 161 CTAs of 12 bursts, and the 13 SMs
      // that hold two of them set its 56 us).  Two CTAs fit an SM; larger grids run in waves of 2 x SMs.
      const double bursts = double(per) / SS_KC > 0.25 ? double(per) / SS_KC : 0.25;
      const double slots = 2.0 * sm_count;
      const double waves = ctas <= 4 * slots ? double(int64_t((ctas + slots - 1) / slots)) : ctas / slots + 0.5;
      t = 5.0e-6 + bursts * (ctas <= sm_count ? 2.67e-6 : waves * 4.36e-6) + (splits > 1 ? 4.0e-6 : 0.0);
    }
    if (best == 0 || t < best) {
      best = t;
      *variant = kVariant[i];
    }
  }
  double biased = best;
  if (sgemm_ffma_supported(A, B, C, N, K)) {
    static const int kPipe[3] = {VT_SGEMM_PIPE128, VT_SGEMM_PIPE64X128, VT_SGEMM_PIPE64};
    for (int shape = 0; shape < 3; ++shape) {
      int splits;
      const double t = sgemm_ffma_plan(c, shape, M, N, K, 0, &splits);
      if (1.05 * t < biased) {                // has to win by 5 % against the kernels before it ...
        biased = 1.05 * t;
        best = t;                             // ... but what the caller compares with other kernels is the estimate itself
        *variant = kPipe[shape];
      }
    }
  }
  return best;
}

int launch_sgemm(DeviceCtx* c, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                 int variant, cudaStream_t s) {
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return fail(VT_ERR_INVALID, "dimension overflows int");
  if (variant == 0) sgemm_tile_choice(c, A, B, C, M, N, K, &variant);
  if (variant == VT_SGEMM_PIPE128 || variant == VT_SGEMM_PIPE64X128 || variant == VT_SGEMM_PIPE64)
    return launch_sgemm_ffma(c, A, B, C, M, N, K, variant == VT_SGEMM_PIPE128 ? 0 : variant == VT_SGEMM_PIPE64X128 ? 1 : 2, s);
  if (variant == VT_SGEMM_TILE32) return launch_small(c, A, B, C, int(M), int(N), int(K), s);
  if (variant == 1) return launch_tile<2, 2>(A, B, C, int(M), int(N), int(K), s);
  if (variant == 2) return launch_tile<1, 1>(A, B, C, int(M), int(N), int(K), s);
  return fail(VT_ERR_UNSUPPORTED, "sgemm variant %d is not built", variant);
}

// ---------------------------------------------------------------------------------------------
// Skinny fp32 GEMM without any allocation.
//
// Some hosts of this library cannot let it allocate device memory: a serving process that has
// handed the whole of HBM to its own pool (PyTorch's caching allocator, an inference runtime with a
// fixed budget) leaves nothing for a library-side cudaMalloc, and where memory is left, cudaMalloc
// still synchronises the device in the middle of a request.  vt_sgemm normally takes the K-split
// partial tiles of the skinny kernel from a grow-only cudaMalloc'd workspace; this entry point takes
// them from the fixed array below instead, which every GPU that loads the library holds until the
// process exits.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchFloats = VT_SKINNY_STATIC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_skinny_static_scratch[kStaticScratchFloats];

struct StaticScratchSlot {
  std::atomic<bool> ready{false};   // published with release once ptr and sm_count are in place
  float* ptr = nullptr;   // device address of g_skinny_static_scratch on this device
  int sm_count = 0;
};
constexpr int kStaticMaxDevices = 16;
StaticScratchSlot g_static_slot[kStaticMaxDevices];
std::mutex g_static_mu;

}  // namespace

}  // namespace vt

extern "C" int vt_sgemm_skinny_static_scratch(int dev, const float* A, const float* B, float* C, int64_t M, int64_t N,
                                              int64_t K, void* stream) {
  using namespace vt;
  clear_error_text();
  if (!A || !B || !C) return fail(VT_ERR_INVALID, "null operand");
  if (dev < 0 || dev >= kStaticMaxDevices) return fail(VT_ERR_INVALID, "device ordinal %d out of range", dev);
  if (M < 1 || N < 1 || K < 1) return fail(VT_ERR_INVALID, "dimensions must be positive");
  if (M > SK_M || N % 4 != 0) return fail(VT_ERR_UNSUPPORTED, "skinny kernel needs M <= 16 and N %% 4 == 0");
  if (N > 0x7fffffffLL || K > 0x7fffffffLL) return fail(VT_ERR_INVALID, "dimension overflows int");
  if ((reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return fail(VT_ERR_INVALID, "B and C must be 16-byte aligned");
  // The launch below goes to `dev`; the caller's current device is put back before returning.
  struct DeviceGuard {
    int prev = -1;
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
  } guard;
  int current = -1;
  VT_CUDA(cudaGetDevice(&current));
  if (current != dev) {
    VT_CUDA(cudaSetDevice(dev));
    guard.prev = current;
  }
  StaticScratchSlot* slot = &g_static_slot[dev];
  if (!slot->ready.load(std::memory_order_acquire)) {
    // Set-up, once per device, with that device current.  In host code the array's name is only
    // a stand-in for the symbol; the address kernels can use comes from the runtime.
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!slot->ready.load(std::memory_order_acquire)) {
      int major = 0, sms = 0;
      VT_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
      if (major != 10)
        return fail(VT_ERR_UNSUPPORTED, "device %d is compute capability %d.x; this library is built for sm_100a only", dev,
                    major);
      float* p = nullptr;
      VT_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_skinny_static_scratch));
      VT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
      if (!p || sms < 1) return fail(VT_ERR_CUDA, "static scratch set-up returned no address");
      slot->ptr = p;
      slot->sm_count = sms;
      slot->ready.store(true, std::memory_order_release);
    }
  }
  int ksplit = 1;
  const size_t need = sgemm_skinny_partials_bytes(M, N, K, slot->sm_count, &ksplit);
  if (need > VT_SKINNY_STATIC_SCRATCH_BYTES)
    return fail(VT_ERR_UNSUPPORTED,
                "%lldx%lldx%lld needs %zu bytes of K-split scratch; the static array holds %zu (use vt_sgemm)",
                (long long)M, (long long)N, (long long)K, need, size_t(VT_SKINNY_STATIC_SCRATCH_BYTES));
  // Every partial cell the reduce pass reads is written by the first pass of this same call, so
  // the previous call's leftovers in the array need no clearing.
  return launch_sgemm_skinny(nullptr, A, B, C, ksplit > 1 ? slot->ptr : nullptr, M, N, K, ksplit,
                             static_cast<cudaStream_t>(stream));
}
