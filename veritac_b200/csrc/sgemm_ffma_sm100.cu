// fp32 GEMM C[M,N] = A[M,K] * B[K,N] in true fp32 arithmetic (FFMA), second design: the loop nest the reference
// emits as OpenMP C (specializations/cpu_gemm/emit_c.py:83-155) with its tiles on CTAs, its reduction loop on a
// software pipeline and, for products of few tiles, split over the CTAs of a thread-block cluster.
//
// The first tile kernels (sgemm_sm100.cu) stay the choice for large products (58 TFLOPS with every SM busy, this
// kernel 54).  What they lack is CTAs when the product is mid-sized: 640^3 is 25 tiles of 128 x 128 or 100 of
// 64 x 64 on 148 SMs.  Here:
//   * operands arrive by cp.async into a ring of kStages stages of 32 values of K, issued two stages ahead, in
//     the layout they have in memory: rows of A are 128 bytes of shared memory whose 16-byte chunks are XOR-ed with
//     the row number (chunk c of row r lies at chunk position c ^ (r & 7)), rows of B lie as they are;
//   * a warp owns 32 rows x 64 columns of the CTA tile as 4 x 8 threads; a thread owns rows 4j + (lane / 8),
//     j = 0..7, and columns 4 (lane % 8) .. +3 of both 32-column halves.  It reads A as float4s along K (eight
//     per four K steps: the four rows a warp reads in one instruction are consecutive, so their chunk positions
//     differ: no bank conflict, measured) and B as two float4s per K step (eight threads read 128 consecutive
//     bytes);
//   * the 8 x 8 outputs of a thread are 32 packed pairs along N, updated by fma.rn.f32x2 with the value of A in
//     both halves of its register pair;
//   * the tile is kWarpsM x kWarpsN warps: 128 x 128 (8 warps, one CTA per SM), 64 x 128 (4 warps, two per SM) or
//     64 x 64 (2 warps, four per SM);
//   * K is split over the CTAs of a thread-block cluster (up to 8) when that fills more of the GPU
//     (sgemm_ffma_plan): every CTA leaves its partial tile in its own shared memory (the ring, idle by then), and
//     after a cluster barrier CTA r adds slice r of all partial tiles, in split order, reading the others' shared
//     memory directly, and writes that slice of C.  The sum does not depend on timing, and no partial tile goes
//     to global memory (through scratch memory and a ticket per tile the adding cost 12-19 us for 64 KiB tiles).
// Needs N % 4 == 0, K % 4 == 0 and 16-byte aligned operands (cp.async moves 16 bytes); M, N, K are otherwise
// free: rows, columns and K values past the edge are zero-filled on the way in and clipped on the way out.
#include "ptx_sm100.cuh"
#include "runtime.h"

namespace vt {
namespace {

constexpr int FF_BK = 32;     // values of K per stage: one 128-byte row of A
constexpr int FF_MAX_CLUSTER = 8;

__device__ __forceinline__ void ff_cp_async_16(uint32_t smem_dst, const float* gmem_src, bool valid) {
  const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ff_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void ff_cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ float4 ff_lds128(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

// The adding of a K split: slice `rank` of the tile (float4s [f_begin, f_end), this thread's every T-th) summed over
// the partial tiles of all CTAs of the cluster, in split order, and written to C.  (A form that issues eight of the
// loads from the other CTAs' shared memory before using the first was measured: the adding is 1-2 us either way,
// and the kernel as a whole came out 4 % slower, K loop included.)
template <int T, int BM, int BN>
__device__ __forceinline__ void ff_add_slices(uint32_t smem0, float* __restrict__ C, int M, int N, int m0, int n0, int splits,
                                           int tid) {
  constexpr int kRowF4 = BN / 4, kTileF4 = BM * kRowF4;
  const int rank = int(cluster_cta_rank());
  const int f_begin = rank * kTileF4 / splits, f_end = (rank + 1) * kTileF4 / splits;
  for (int f = f_begin + tid; f < f_end; f += T) {
    float4 sum = ld_shared_cluster_v4f(mapa_shared(smem0 + uint32_t(f) * 16u, 0));
    for (int q = 1; q < splits; ++q) {
      const float4 v = ld_shared_cluster_v4f(mapa_shared(smem0 + uint32_t(f) * 16u, uint32_t(q)));
      sum.x += v.x;
      sum.y += v.y;
      sum.z += v.z;
      sum.w += v.w;
    }
    const int row = m0 + f / kRowF4, col = n0 + (f % kRowF4) * 4;
    if (row < M && col < N) *reinterpret_cast<float4*>(C + size_t(row) * N + col) = sum;
  }
}

template <int kWarpsM, int kWarpsN, int kStages>
struct FfShape {
  static constexpr int kThreads = kWarpsM * kWarpsN * 32;
  static constexpr int BM = kWarpsM * 32, BN = kWarpsN * 64;
  static constexpr int kABytes = BM * FF_BK * 4, kBBytes = FF_BK * BN * 4;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTileBytes = BM * BN * 4;
  static constexpr int kSmemBytes = kStages * kStageBytes > kTileBytes ? kStages * kStageBytes : kTileBytes;
  // Eight warps per SM: the 8 x 8 outputs and the eight float4s of A a thread holds take ~170 registers.  (Reading A
  // two values of K at a time fits 128 registers and sixteen warps per SM; measured slower, 21.0 against 20.5 ms at
  // 8192^3: twice the loads of A.)
  static constexpr int kCtasBySmem = (227 * 1024) / (kSmemBytes + 1024);
  static constexpr int kCtasByWarps = 8 / (kWarpsM * kWarpsN) < 1 ? 1 : 8 / (kWarpsM * kWarpsN);
  static constexpr int kCtasPerSm = kCtasByWarps < kCtasBySmem ? kCtasByWarps : kCtasBySmem;
};

template <int kWarpsM, int kWarpsN, int kStages>
__global__ void __launch_bounds__(FfShape<kWarpsM, kWarpsN, kStages>::kThreads, FfShape<kWarpsM, kWarpsN, kStages>::kCtasPerSm)
sgemm_ffma_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N, int K,
                  int tiles_m, int tiles_n, int group, int splits, int k_per_split) {
  using S = FfShape<kWarpsM, kWarpsN, kStages>;
  constexpr int T = S::kThreads, BM = S::BM, BN = S::BN;
  extern __shared__ __align__(128) uint8_t ff_smem[];
  const uint32_t smem0 = smem_u32(ff_smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int warp_m = warp / kWarpsN, warp_n = warp - warp_m * kWarpsN;
  const int ty = lane >> 3, tx = lane & 7;

  // Tile and K range.  The CTAs of one tile are consecutive (one cluster when K is split); tiles go in the grouped
  // order of the first kernel: all tile-columns for `group` tile-rows at a time.
  const int tile = blockIdx.x / splits;
  const int k_begin = (blockIdx.x - tile * splits) * k_per_split;
  const int k_end = min(K, k_begin + k_per_split);
  int tm, tn;
  {
    const int per = group * tiles_n;
    const int g = tile / per;
    const int w = tile - g * per;
    const int rows = min(group, tiles_m - g * group);
    tn = w / rows;
    tm = g * group + (w - tn * rows);
  }
  const int m0 = tm * BM, n0 = tn * BN;
  const int nk = (k_end - k_begin + FF_BK - 1) / FF_BK;

  // Copies of one stage: A is BM rows x 8 chunks, B is 32 rows x BN / 4 chunks.
  constexpr int kACopies = BM * 8 / T, kBCopies = FF_BK * (BN / 4) / T;
  auto load_stage = [&](int kt) {
    const int k0 = k_begin + kt * FF_BK;
    const uint32_t a_s = smem0 + uint32_t(kt % kStages) * S::kStageBytes, b_s = a_s + S::kABytes;
#pragma unroll
    for (int i = 0; i < kACopies; ++i) {
      const int f = tid + T * i;
      const int row = f >> 3, c = f & 7;
      const bool ok = (m0 + row < M) && (k0 + c * 4 < k_end);
      ff_cp_async_16(a_s + uint32_t(row * 128 + ((c ^ (row & 7)) << 4)), ok ? A + size_t(m0 + row) * K + k0 + c * 4 : A, ok);
    }
#pragma unroll
    for (int i = 0; i < kBCopies; ++i) {
      const int f = tid + T * i;
      const int row = f / (BN / 4), c4 = f - row * (BN / 4);
      const bool ok = (k0 + row < k_end) && (n0 + c4 * 4 < N);
      ff_cp_async_16(b_s + uint32_t(row * (BN * 4) + c4 * 16), ok ? B + size_t(k0 + row) * N + n0 + c4 * 4 : B, ok);
    }
  };

  // acc[j][q]: row 4j + ty of the warp's 32, column pair q of the thread's eight columns.
  float2 acc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[j][q] = make_float2(0.f, 0.f);

  // Launched for overlap with the kernel before it on the stream: nothing is read or written before it has completed.
  grid_dependency_wait();
  grid_launch_dependents();

#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < nk) load_stage(s);
    ff_cp_async_commit();
  }

  // Row j of this thread lies at byte (warp_m * 32 + 4j + ty) * 128 of a stage's A; its chunk positions are XOR-ed
  // with (4j + ty) & 7 = 4 (j & 1) + ty.
  const uint32_t a_row0 = uint32_t((warp_m * 32 + ty) * 128);
  const uint32_t swz_even = uint32_t(ty) << 4, swz_odd = uint32_t(4 + ty) << 4;
  const uint32_t b_col0 = uint32_t(S::kABytes + (warp_n * 64 + tx * 4) * 4);

  for (int kt = 0; kt < nk; ++kt) {
    ff_cp_async_wait<kStages - 2>();      // this thread's copies of stage kt have landed
    __syncthreads();                      // ... and everyone's; and everyone is done with stage kt - 1
    if (kt + kStages - 1 < nk) load_stage(kt + kStages - 1);
    ff_cp_async_commit();
    const uint32_t stage = smem0 + uint32_t(kt % kStages) * S::kStageBytes;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float4 a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        a[j] = ff_lds128(stage + a_row0 + uint32_t(j * 512) + ((uint32_t(c) << 4) ^ ((j & 1) ? swz_odd : swz_even)));
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint32_t b_addr = stage + b_col0 + uint32_t((c * 4 + kk) * (BN * 4));
        const float4 b0 = ff_lds128(b_addr), b1 = ff_lds128(b_addr + 128);
        const float2 bp[4] = {make_float2(b0.x, b0.y), make_float2(b0.z, b0.w), make_float2(b1.x, b1.y),
                              make_float2(b1.z, b1.w)};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float av = kk == 0 ? a[j].x : kk == 1 ? a[j].y : kk == 2 ? a[j].z : a[j].w;
          const float2 ad = make_float2(av, av);
#pragma unroll
          for (int q = 0; q < 4; ++q) acc[j][q] = __ffma2_rn(ad, bp[q], acc[j][q]);
        }
      }
    }
  }

  if (splits == 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int row = m0 + warp_m * 32 + 4 * j + ty;
      if (row < M) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int col = n0 + warp_n * 64 + 32 * h + tx * 4;
          if (col < N)
            *reinterpret_cast<float4*>(C + size_t(row) * N + col) =
                make_float4(acc[j][2 * h].x, acc[j][2 * h].y, acc[j][2 * h + 1].x, acc[j][2 * h + 1].y);
        }
      }
    }
    return;
  }

  // K split over the cluster: partial tile into the ring (row-major, BN floats per row), barrier, every CTA adds
  // its slice of all partial tiles in split order.
  ff_cp_async_wait<0>();
  __syncthreads();                        // everyone is done reading the ring
  constexpr int kRowF4 = BN / 4;
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t f = uint32_t((warp_m * 32 + 4 * j + ty) * kRowF4 + warp_n * 16 + 8 * h + tx);
      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(smem0 + f * 16u), "f"(acc[j][2 * h].x),
                   "f"(acc[j][2 * h].y), "f"(acc[j][2 * h + 1].x), "f"(acc[j][2 * h + 1].y)
                   : "memory");
    }
  cluster_sync_all();
  ff_add_slices<T, BM, BN>(smem0, C, M, N, m0, n0, splits, tid);
  cluster_sync_all();                     // nobody leaves while its shared memory may still be read
}

template <int kWarpsM, int kWarpsN, int kStages>
int launch_ffma(DeviceCtx* c, const float* A, const float* B, float* C, int M, int N, int K, int splits, cudaStream_t s) {
  using S = FfShape<kWarpsM, kWarpsN, kStages>;
  const int tiles_m = (M + S::BM - 1) / S::BM, tiles_n = (N + S::BN - 1) / S::BN;
  const long long tiles = 1LL * tiles_m * tiles_n;
  const int group = tiles_m < 8 ? tiles_m : 8;
  int k_per_split;
  {
    const int steps = (K + FF_BK - 1) / FF_BK;
    const int per = (steps + splits - 1) / splits;
    k_per_split = per * FF_BK;
    splits = (steps + per - 1) / per;
  }
  if (tiles * splits > 0x7fffffffLL) return fail(VT_ERR_INVALID, "sgemm tile count overflows int");
  auto kernel = sgemm_ffma_kernel<kWarpsM, kWarpsN, kStages>;
  (void)c;      // the kernel's shared-memory opt-in was set on this device when its cluster capacities were queried
  if (splits > 1)
    VT_CUDA(launch_overlapped_cluster(kernel, unsigned(tiles * splits), unsigned(S::kThreads), size_t(S::kSmemBytes),
                                      unsigned(splits), s, A, B, C, M, N, K, tiles_m, tiles_n, group, splits, k_per_split));
  else
    VT_CUDA(launch_overlapped(kernel, unsigned(tiles), unsigned(S::kThreads), size_t(S::kSmemBytes), s, A, B, C, M, N, K,
                              tiles_m, tiles_n, group, splits, k_per_split));
  count_launch();
  VT_CUDA(cudaGetLastError());
  return VT_OK;
}

// The three tile shapes that are built (index = `shape` below).
template <int kShape> struct FfPick;
template <> struct FfPick<0> { using S = FfShape<4, 2, 3>; static constexpr int WM = 4, WN = 2; };   // 128 x 128
template <> struct FfPick<1> { using S = FfShape<2, 2, 3>; static constexpr int WM = 2, WN = 2; };   // 64 x 128
template <> struct FfPick<2> { using S = FfShape<2, 1, 3>; static constexpr int WM = 2, WN = 1; };   // 64 x 64

// How many clusters of `size` CTAs of a shape the device holds at once (a cluster lives inside one GPC, so this
// is not SMs / size: 128 x 128 tiles, one CTA per SM: 148, 74, 45, 33, 26, 22, 15, 15 for sizes 1 to 8).
template <int kShape>
int cluster_capacity(int size) {
  using S = typename FfPick<kShape>::S;
  auto kernel = sgemm_ffma_kernel<FfPick<kShape>::WM, FfPick<kShape>::WN, 3>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(S::kSmemBytes)) != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(size) * 64);
  cfg.blockDim = dim3(S::kThreads);
  cfg.dynamicSmemBytes = S::kSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = unsigned(size);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

void fill_capacity(DeviceCtx* c) {
  if (c->ffma_capacity_known) return;
  for (int size = 1; size <= FF_MAX_CLUSTER; ++size) {
    c->ffma_capacity[0][size] = cluster_capacity<0>(size);
    c->ffma_capacity[1][size] = cluster_capacity<1>(size);
    c->ffma_capacity[2][size] = cluster_capacity<2>(size);
  }
  c->ffma_capacity_known = true;
}

}  // namespace

bool sgemm_ffma_supported(const float* A, const float* B, const float* C, int64_t N, int64_t K) {
  return N % 4 == 0 && K % 4 == 0 &&
         ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) == 0;
}

// Modelled time (seconds) of tile shape `shape` on an M x N x K product, and the K split it is reached with.
// An SM with eight resident warps of this kernel completes one 128 x 128 x 32 step's worth of FMAs in 2.87 us
// (measured; 74 % of the FMA pipe); with six warps (two of the four schedulers hold two) it runs at 0.75 of that
// rate, with four at 0.84, with two at 0.46.  A launch costs about 5 us beside its K loop (launch, first loads,
// last stores) and a split 2 us more (cluster barriers and the adding).  Candidates are the splits 1..8 whose
// clusters the device can hold (cluster_capacity); a grid larger than the capacity runs in waves.  Where the CTAs
// land: a cluster stays inside one GPC, clusters are dealt over the eight GPCs of about 19 SMs, and CTAs share an SM
// once the clusters of a GPC hold more CTAs than it has SMs, or the grid more CTAs than the clusters of that size
// reach SMs (the capacity of the one-CTA-per-SM shape).  Against a sweep of 28 mid-sized shapes x 3 tile shapes x
// 8 splits the model's r.m.s. error is 10 %, and choosing by it costs 2 % against the best measured candidate.
double sgemm_ffma_plan(DeviceCtx* c, int shape, int64_t M, int64_t N, int64_t K, int forced, int* splits_out) {
  fill_capacity(c);
  const int bm = shape == 0 ? 128 : 64, bn = shape == 2 ? 64 : 128, warps_cta = bm * bn / 2048;
  const int resident_most = shape == 0 ? 1 : shape == 1 ? 2 : 4;
  const double tiles = double((M + bm - 1) / bm) * double((N + bn - 1) / bn);
  const int64_t steps_total = (K + FF_BK - 1) / FF_BK;
  double best = 0;
  *splits_out = 1;
  for (int want = 1; want <= FF_MAX_CLUSTER; ++want) {
    if (forced > 0 && want != (forced > FF_MAX_CLUSTER ? FF_MAX_CLUSTER : forced)) continue;
    const int64_t per = (steps_total + want - 1) / want;
    const int s = int((steps_total + per - 1) / per);
    if (s != want && forced <= 0) continue;                  // the same split as a smaller `want`
    if (s > 1 && per < 2 && forced <= 0) continue;
    // One cluster fewer than the occupancy query promises when K is split: a grid that needs every last one did not
    // get them in one wave (45 clusters of three 128 x 128 CTAs, capacity 45: 85 us where one wave would be 64).
    const double capacity = double(c->ffma_capacity[shape][s] - (s > 1 ? 1 : 0)) * s;
    const double reach = double(c->ffma_capacity[0][s]) * s;
    if (capacity <= 0 || reach <= 0) continue;
    const double ctas = tiles * s;
    const double waves = ctas <= capacity ? 1.0 : double(int64_t((ctas + capacity - 1) / capacity));
    const double in_wave = ctas < capacity ? ctas : capacity;
    double per_sm = double(int64_t((in_wave + reach - 1) / reach));
    if (s > 1) {
      const double per_gpc = double(int64_t((in_wave / s + 7) / 8)) * s;
      const double crowded = double(int64_t((per_gpc + 18) / 19));
      if (crowded > per_sm) per_sm = crowded;
    }
    if (per_sm > resident_most) per_sm = resident_most;
    const double warps = per_sm * warps_cta;
    const double rate = warps >= 8 ? 1.0 : warps >= 6 ? 0.75 : warps >= 4 ? 0.84 : 0.46;
    const double step = per_sm * (double(bm) * bn / 16384.0) * 2.87e-6 / rate;
    const double t = 5.0e-6 + waves * (double(per) * step + (s > 1 ? 2.0e-6 : 0.0));
    if (best == 0 || t < best) {
      best = t;
      *splits_out = s;
    }
  }
  if (best == 0) best = 1.0e9;
  return best;
}

int launch_sgemm_ffma(DeviceCtx* c, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int shape,
                      cudaStream_t s) {
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return fail(VT_ERR_INVALID, "dimension overflows int");
  if (!sgemm_ffma_supported(A, B, C, N, K))
    return fail(VT_ERR_UNSUPPORTED, "the pipelined FFMA kernel needs N %% 4 == 0, K %% 4 == 0 and 16-byte aligned operands");
  int splits = 1;
  sgemm_ffma_plan(c, shape, M, N, K, c->sgemm_force_splits > 0 ? c->sgemm_force_splits : 0, &splits);
  if (shape == 0) return launch_ffma<4, 2, 3>(c, A, B, C, int(M), int(N), int(K), splits, s);
  if (shape == 1) return launch_ffma<2, 2, 3>(c, A, B, C, int(M), int(N), int(K), splits, s);
  return launch_ffma<2, 1, 3>(c, A, B, C, int(M), int(N), int(K), splits, s);
}

}  // namespace vt
