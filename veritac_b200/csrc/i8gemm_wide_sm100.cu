// Exact int8 x int8 -> int32 GEMM, CTA pairs on 256 x 512 output tiles ("wide" form of the pair kernel in
// i8gemm_sm100.cu; same arithmetic, same reference lines: specializations/gemmini_gemm/backend.py:490-529).
//
// Why a second form.  With the SM clock high (launches of tens of microseconds, before the power cap bites) the
// 256 x 256 pair kernel is bound by what the L2 can deliver to the SMs, not by the tensor pipe: per K block of 128
// a pair fetches 64 KiB for 256 x 256 x 128 products.  Two neighbouring tiles of one tile-row need the same 256
// rows of A.  Here a pair computes both at once: one stage holds the pair's 256 x 128 block of A and two
// 128 x 256 blocks of B (48 KiB per CTA), and every K step issues one MMA per half into its own 256-column TMEM
// accumulator, so 96 KiB are fetched for twice the products: a quarter less L2 traffic per product, which makes
// the tensor pipe the limit again.  Tensor memory is then full (2 x 256 columns, both live), so the epilogue of a
// tile cannot overlap the MMAs of the next one; the form pays where a pair has few tiles (row shards of a
// multi-GPU job, products of a few hundred tiles) and loses to the double-buffered kernel on long runs, where
// the power cap, not the L2, sets the pace.  Measured figures are with the launcher's choice in capi.cu.
//
// Structure as the pair kernel: warp 0 of each CTA loads (TMA, 128-byte swizzle, B as stored), warp 1 of the even
// CTA issues tcgen05.mma.cta_group::2.kind::i8 (M = 256, N = 256, K = 32), eight epilogue warps per CTA move
// 32 rows x 256 columns each from TMEM through swizzled shared memory to TMA stores.  Every wait is bounded; a
// pair that gives up settles its barriers and waits for copies in flight before it leaves (pair_drain_loads).
#include "ptx_sm100.cuh"
#include "runtime.h"
#include "umma_tile.cuh"

namespace vt {
namespace {

constexpr int W_BK = 128;                           // int8 elements == bytes: one 128-byte swizzle row of K
constexpr int W_UMMA_K = 32;
constexpr int W_STAGES = 4;
constexpr int W_EPI_WARPS = 8;                      // two per TMEM lane quarter: one per half of the wide tile
constexpr int W_THREADS = 32 * (2 + W_EPI_WARPS);   // 1 TMA warp, 1 MMA warp, the epilogue warps
constexpr int W_WARP_CHUNKS = 16 / (W_EPI_WARPS / 4);   // 32-column chunks of the two accumulators one warp moves
constexpr int W_WIDE_BUFS = 48 / W_EPI_WARPS;       // store buffers per warp that the idle operand ring (192 KiB) provides
static_assert(W_EPI_WARPS == 4 || W_EPI_WARPS == 8, "one or two epilogue warps per TMEM lane quarter");
constexpr int W_A_BYTES = 128 * W_BK;               // this CTA's 128 rows of A
constexpr int W_B_BYTES = 128 * W_BK;               // this CTA's 128 columns of one half's B
constexpr int W_STAGE_BYTES = W_A_BYTES + 2 * W_B_BYTES;   // 48 KiB
constexpr int W_TILE_N = 512;

struct WidePipeState {
  uint64_t full[W_STAGES];
  uint64_t empty[W_STAGES];
  uint64_t tmem_full;
  uint64_t tmem_empty;
  uint32_t tmem_base;
  int abort_word;
  uint32_t peer_abort;
  uint32_t fills_own;
  uint32_t fills_peer;
};

constexpr size_t WIDE_SMEM_BYTES = 1024 + size_t(W_STAGES) * W_STAGE_BYTES + size_t(W_EPI_WARPS) * EPI_BUF_BYTES + 256;
static_assert(sizeof(WidePipeState) <= 256, "pipeline state outgrew its shared-memory reserve");

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(W_THREADS, 1)
i8gemm_umma_pair_wide_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                             const __grid_constant__ CUtensorMap tmC, int M, int N, int K, TileRaster rs,
                             int* __restrict__ status, long long wait_limit) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = tiles + size_t(W_STAGES) * W_STAGE_BYTES;
  const uint64_t store_policy = l2_policy_evict_first();   // C is written once and never read here
  WidePipeState* ps = reinterpret_cast<WidePipeState*>(staging + W_EPI_WARPS * EPI_BUF_BYTES);
  volatile int* abort_word = &ps->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();          // 0 = even CTA (issues the MMAs), 1 = its peer
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = rs.mt * rs.nt;               // 256 x 512 tiles
  const int kblocks = (K + W_BK - 1) / W_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < W_STAGES; ++s) {
      mbar_init(&ps->full[s], 1);                    // the even CTA's producer arrives (with both CTAs' bytes)
      mbar_init(&ps->empty[s], 1);                   // one multicast commit
    }
    mbar_init(&ps->tmem_full, 1);                    // one multicast commit
    mbar_init(&ps->tmem_empty, 2 * W_EPI_WARPS);     // the epilogue warps of both CTAs
    ps->abort_word = 0;
    ps->peer_abort = 0;
    ps->fills_own = 0;
    ps->fills_peer = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc<2>(&ps->tmem_base, TMEM_COLS);
    tmem_relinquish<2>();
  }
  tc_fence_before_sync();
  cluster_sync_all();                                // peer barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = ps->tmem_base;
  // The set-up above may overlap the end of the kernel before this one on the stream; operands, C and the
  // status word are not touched before that kernel has completed.
  grid_dependency_wait();
  grid_launch_dependents();

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, fills = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int mi, ni;
        tile_coords(rs, t, mi, ni);
        const int m0 = mi * 256 + int(rank) * 128, n0 = ni * W_TILE_N + int(rank) * 128;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&ps->empty[stage], phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_PRODUCER, wait_limit)) {
            ok = false;
            break;
          }
          uint8_t* a_s = tiles + size_t(stage) * W_STAGE_BYTES;
          if (rank == 0) mbar_arrive_expect_tx(&ps->full[stage], 2 * W_STAGE_BYTES);
          const uint32_t full_even = mapa_shared(smem_u32(&ps->full[stage]), 0);
          tma_load_2d_pair(a_s, &tmA, full_even, kb * W_BK, m0);
          tma_load_2d_pair(a_s + W_A_BYTES, &tmB, full_even, n0, kb * W_BK);                   // left half's columns
          tma_load_2d_pair(a_s + W_A_BYTES + W_B_BYTES, &tmB, full_even, n0 + 256, kb * W_BK);   // right half's
          ++fills;
          if (++stage == W_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (ok) {
        // Every stage released => every MMA that reads shared memory has retired before the ring is reused by
        // the last epilogue or given back.
        for (int s = 0; s < W_STAGES; ++s) {
          if (!mbar_wait(&ps->empty[stage], phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_PRODUCER, wait_limit)) break;
          if (++stage == W_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (rank == 0) ps->fills_own = fills;
      else st_shared_cluster_u32(mapa_shared(smem_u32(&ps->fills_peer), 0), fills);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA only) ------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_instr_desc(UMMA_D_S32, UMMA_AB_S8, false, true, 256, 256);
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        if (!mbar_wait<true>(&ps->tmem_empty, acc_phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_MMA, wait_limit)) break;
        tc_fence_after_sync();
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait<true>(&ps->full[stage], phase, abort_word, KSTAT_WAIT_EXPIRED_MMA, wait_limit)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(tiles + size_t(stage) * W_STAGE_BYTES);
          const uint32_t b_addr = a_addr + W_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < W_BK / W_UMMA_K; ++kk) {
            // A: K-major, 32 bytes per K step inside the swizzle row.  B as stored (N contiguous): each CTA holds
            // one 128-column box per half, the pair's two boxes form the 256 columns; a K step of 32 rows moves 4 KiB.
            const uint64_t a_desc = umma_smem_desc_sw128(a_addr + kk * W_UMMA_K, 16, 1024);
            const uint64_t b0_desc = umma_smem_desc_sw128(b_addr + kk * W_UMMA_K * 128, W_B_BYTES, 1024);
            const uint64_t b1_desc = umma_smem_desc_sw128(b_addr + W_B_BYTES + kk * W_UMMA_K * 128, W_B_BYTES, 1024);
            umma_i8<2>(tmem_base, a_desc, b0_desc, idesc, uint32_t((kb | kk) != 0));
            umma_i8<2>(tmem_base + 256u, a_desc, b1_desc, idesc, uint32_t((kb | kk) != 0));
          }
          umma_commit_pair(&ps->empty[stage], 3);
          if (++stage == W_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair(&ps->tmem_full, 3);
        acc_phase ^= 1;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue (both CTAs, 8 warps) ------------------------------
    // Epilogue warp e owns TMEM lane quarter (warp % 4) and, with two warps per quarter, one half of the wide tile.
    const int e = warp - 2;
    const int q = warp & 3;
    const int c_begin = (e >> 2) * W_WARP_CHUNKS, c_end = c_begin + W_WARP_CHUNKS;
    uint32_t acc_phase = 0;
    for (int t = pair; t < num_tiles; t += num_pairs) {
      int mi, ni;
      tile_coords(rs, t, mi, ni);
      const int m0 = mi * 256 + int(rank) * 128, n0 = ni * W_TILE_N;
      const bool ready = mbar_wait<true>(&ps->tmem_full, acc_phase, abort_word, KSTAT_WAIT_EXPIRED_EPILOGUE, wait_limit);
      if (!__all_sync(0xffffffffu, ready)) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16);
      // After the pair's last tile every MMA has read its operands and no load is in flight: the operand ring then
      // serves as store buffers (192 KiB shared out between the warps), so that few stores wait for a buffer.
      uint8_t* wide = t + num_pairs >= num_tiles ? tiles + size_t(e) * W_WIDE_BUFS * EPI_BUF_BYTES : nullptr;
      epilogue_warp_tile<1, W_WIDE_BUFS>(t_row, &tmC, staging + e * EPI_BUF_BYTES, M, N, m0 + q * 32, n0, lane, store_policy, wide,
                                         c_begin, c_end);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(&ps->tmem_empty, 0);
      acc_phase ^= 1;
    }
    // The stores have read their shared-memory buffers; the writes themselves complete before the grid does.
    if (lane == 0) tma_store_wait_read<0>();
    __syncwarp();
  }

  // Neither CTA may free TMEM or leave while its peer's MMAs, commits or remote arrivals can still touch it; a pair
  // that gave up first makes sure that no copy is still on its way into either CTA's shared memory.
  tc_fence_before_sync();
  __syncthreads();                                   // every role of this CTA is done: the abort word is final
  if (threadIdx.x == 0)
    st_shared_cluster_u32(mapa_shared(smem_u32(&ps->peer_abort), rank ^ 1u), uint32_t(ps->abort_word));
  cluster_sync_all();
  if (ps->abort_word != 0 || ps->peer_abort != 0) {  // the same verdict in both CTAs
    if (rank == 0 && threadIdx.x == 0 &&
        !pair_drain_loads<W_STAGES>(ps->full, ps->fills_own, ps->fills_peer, W_STAGE_BYTES))
      atomicCAS(&ps->abort_word, 0, KSTAT_WAIT_EXPIRED_DRAIN);
    cluster_sync_all();
  }
  if (warp == 1) tmem_dealloc<2>(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && ps->abort_word != 0) atomicCAS(status, 0, ps->abort_word);
}

}  // namespace

int launch_i8gemm_wide(DeviceCtx* c, const int8_t* A, const int8_t* B, int32_t* C, int64_t M, int64_t N, int64_t K,
                       int raster_mode, int group, cudaStream_t s, int64_t ldb, int64_t ldc) {
  if (ldb == 0) ldb = N;
  if (ldc == 0) ldc = N;
  if (ldb < N || ldc < N || (ldb & 15) || (ldc & 3)) return fail(VT_ERR_INVALID, "bad row pitch for B or C");
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return fail(VT_ERR_INVALID, "i8gemm operands must be 16-byte aligned");
  if (raster_mode < 0 || raster_mode > 2) return fail(VT_ERR_INVALID, "raster mode %d out of range", raster_mode);
  TileRaster rs;
  rs.mt = int((M + 255) / 256);
  rs.nt = int((N + W_TILE_N - 1) / W_TILE_N);
  rs.mode = raster_mode;
  const int g = (group + 1) / 2;                   // `group` counts 128-row tile-rows
  rs.group = g < 1 ? 1 : (g > rs.mt ? rs.mt : g);
  const long long tiles = 1LL * rs.mt * rs.nt;
  if (tiles > 0x7fffffffLL) return fail(VT_ERR_INVALID, "tile count overflows int");
  CUtensorMap tmA, tmB, tmC;
  int rc = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, uint64_t(K), uint64_t(M), uint64_t(K), W_BK, 128);
  if (rc) return rc;
  rc = encode_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, C, uint64_t(N), uint64_t(M), uint64_t(ldc) * 4, 32, 32);
  if (rc) return rc;
  rc = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, uint64_t(N), uint64_t(K), uint64_t(ldb), 128, W_BK);
  if (rc) return rc;
  const int max_pairs = c->sm_count / 2;
  const int pairs = int(tiles < max_pairs ? tiles : max_pairs);
  if (!(c->func_attr_mask & 2u)) {
    VT_CUDA(cudaFuncSetAttribute(i8gemm_umma_pair_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(WIDE_SMEM_BYTES)));
    c->func_attr_mask |= 2u;
  }
  VT_CUDA(launch_overlapped(i8gemm_umma_pair_wide_kernel, unsigned(2 * pairs), unsigned(W_THREADS), WIDE_SMEM_BYTES, s, tmA,
                            tmB, tmC, int(M), int(N), int(K), rs, c->status, c->wait_limit_cycles));
  count_launch();
  VT_CUDA(cudaGetLastError());
  return VT_OK;
}

}  // namespace vt
