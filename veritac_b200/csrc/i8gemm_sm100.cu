// Exact int8 x int8 -> int32 GEMM for sm_100a: C[M,N] = A[M,K] * B[K,N], all row-major.
//
// This is the arithmetic of the Gemmini full-tile GEMM (a DIM=16 systolic array that overwrites an
// accumulator tile at the first K tile and accumulates onto it afterwards, reference
// specializations/gemmini_gemm/backend.py:490-529) executed on the 5th-generation tensor cores.
// Under the plan's bound k*16384 <= 2^31-1 no partial sum can leave int32, so summation order is
// unobservable and the result is bit-exact for every schedule (VeriTac/GemminiExact.lean:62-75).
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: 128x128 int8 tile of A (K-major, 128-byte swizzle) and a 128(K)x256(N)
//               slab of B exactly as stored (N contiguous => "MN-major" operand, two 128-column boxes),
//               into a shared-memory ring guarded by full/empty mbarriers.
//   warp 1      MMA issuer: one thread issues tcgen05.mma.kind::i8 (K=32) four times per stage into one
//               of two 256-column TMEM accumulators; tcgen05.commit releases the stage and, after the
//               last K block, publishes the accumulator.
//   warps 2..5  epilogue: tcgen05.ld the accumulator quarter owned by (warp % 4), stage it in swizzled
//               shared memory, TMA-store int32 rows to HBM, then hand the accumulator back so the next
//               tile's MMAs overlap.
// Tiles are visited in the order the Gemmini schedule implies (row-major for baseline i,j,k,
// column-major for reuse_b j,k,i, grouped for the batched B-reuse lowering); the order changes L2
// reuse only, never results.
#include "ptx_sm100.cuh"
#include "runtime.h"
#include "umma_tile.cuh"

namespace vt {
namespace {

constexpr int BM = 128;
constexpr int BK = 128;  // int8 elements == bytes: one 128-byte swizzle row of K
constexpr int UMMA_K = 32;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK;              // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK;              // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int B_BOX_BYTES = 128 * BK;               // one 128-column box of the B slab

struct PipeState {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_word;
};

constexpr size_t SMEM_BYTES = 1024 + size_t(STAGES) * STAGE_BYTES + EPI_STAGING_BYTES + sizeof(PipeState);

// One CTA per 128 x 256 tile; tmB describes B as stored (inner = N, outer = K).
__global__ void __launch_bounds__(NUM_THREADS, 1)
i8gemm_umma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmC, int M, int N, int K, TileRaster rs,
                   int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = tiles + size_t(STAGES) * STAGE_BYTES;
  PipeState* ps = reinterpret_cast<PipeState*>(staging + EPI_STAGING_BYTES);
  volatile int* abort_word = &ps->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = rs.mt * rs.nt;
  const int kblocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ps->full[s], 1);
      mbar_init(&ps->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&ps->tmem_full[b], 1);
      mbar_init(&ps->tmem_empty[b], 4);  // one arrival per epilogue warp
    }
    ps->abort_word = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc<1>(&ps->tmem_base, TMEM_COLS);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ps->tmem_base;
  grid_dependency_wait();                            // see the CTA-pair kernel
  grid_launch_dependents();

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t filled = 0, fill_parity = 0;  // per-stage bookkeeping for the abort drain
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mi, ni;
        tile_coords(rs, t, mi, ni);
        const int m0 = mi * BM, n0 = ni * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&ps->empty[stage], phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_PRODUCER)) {
            ok = false;
            break;
          }
          uint64_t* full = &ps->full[stage];
          uint8_t* a_s = tiles + size_t(stage) * STAGE_BYTES;
          uint8_t* b_s = a_s + A_STAGE_BYTES;
          mbar_arrive_expect_tx(full, STAGE_BYTES);
          tma_load_2d(a_s, &tmA, full, kb * BK, m0);
          tma_load_2d(b_s, &tmB, full, n0, kb * BK);
          tma_load_2d(b_s + B_BOX_BYTES, &tmB, full, n0 + 128, kb * BK);
          filled |= 1u << stage;
          fill_parity = (fill_parity & ~(1u << stage)) | (phase << stage);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (ok) {
        // Tail: every stage released => every MMA that reads shared memory has retired and every
        // commit arrival has landed before the CTA gives its shared memory back.
        for (int s = 0; s < STAGES; ++s) {
          if (!mbar_wait(&ps->empty[stage], phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_PRODUCER)) break;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (*abort_word != 0) {
        // Aborting: wait (bounded, ignoring the abort word) for copies already issued to land.
        for (int s = 0; s < STAGES; ++s)
          if (filled & (1u << s)) mbar_wait_drain(&ps->full[s], (fill_parity >> s) & 1u);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_instr_desc(UMMA_D_S32, UMMA_AB_S8, false, true, BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&ps->tmem_empty[acc], acc_phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_MMA)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + uint32_t(acc * BN);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&ps->full[stage], phase, abort_word, KSTAT_WAIT_EXPIRED_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(tiles + size_t(stage) * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // A: K-major, rows of 128 bytes, 8-row groups 1024 bytes apart; a K step of 32 moves 32 bytes
            // inside the swizzle row.
            const uint64_t a_desc = umma_smem_desc_sw128(a_addr + kk * UMMA_K, 16, 1024);
            // B as stored: N contiguous.  128-column blocks are one TMA box (16 KiB) apart,
            // 8-row K groups 1024 bytes apart; a K step of 32 rows moves 4096 bytes.
            const uint64_t b_desc = umma_smem_desc_sw128(b_addr + kk * UMMA_K * 128, B_BOX_BYTES, 1024);
            umma_i8<1>(d_tmem, a_desc, b_desc, idesc, uint32_t((kb | kk) != 0));
          }
          umma_commit(&ps->empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&ps->tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int mi, ni;
      tile_coords(rs, t, mi, ni);
      const int m0 = mi * BM, n0 = ni * BN;
      const bool ready = mbar_wait(&ps->tmem_full[acc], acc_phase, abort_word, KSTAT_WAIT_EXPIRED_EPILOGUE);
      if (!__all_sync(0xffffffffu, ready)) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * BN);
      epilogue_warp_tile<2>(t_row, &tmC, staging + q * 2 * EPI_BUF_BYTES, M, N, m0 + q * 32, n0, lane);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ps->tmem_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    // The stores have read their shared-memory buffers; the writes themselves complete before the grid does.
    if (lane == 0) tma_store_wait_read<0>();
    __syncwarp();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc<1>(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && ps->abort_word != 0) atomicCAS(status, 0, ps->abort_word);
}

// ---------------------------------------------------------------------------------------------
// CTA-pair form (tcgen05 cta_group::2): two CTAs of a 2-cluster, on the two SMs of one TPC, own one
// 256 x 256 output tile.  CTA r holds rows [128r, 128r+128) of the A tile and columns
// [128r, 128r+128) of the B slab in its own shared memory (32 KiB per stage instead of 48, so six
// stages fit) and its own 128 x 256 half of the accumulator in its own TMEM; the MMA instruction,
// issued by the even CTA only, reads both halves of both operands.  Per SM and per K block this
// moves a third less operand data through the L2 -> SM path than the single-CTA form.
//   * both producers signal the even CTA's "full" barrier (it expects both CTAs' bytes);
//   * tcgen05.commit multicasts the "empty" and "accumulator full" arrivals to both CTAs;
//   * both CTAs' epilogue warps arrive on the even CTA's "accumulator empty" barrier (8 arrivals).
// Tiles go to the pairs round-robin, a whole tile at a time.  (Sharing the K blocks of a last, partial round of tiles
// between the pairs was built three ways, bit-exact, and measured level: while some pairs idle the others run their
// K blocks faster, so a half-empty last round costs little.)
// ---------------------------------------------------------------------------------------------
constexpr int P_A_BYTES = 128 * BK;                 // this CTA's 128 rows of A
constexpr int P_B_BYTES = 128 * BK;                 // this CTA's 128 columns of B (one TMA box)
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_STAGES = 6;
// Epilogue warps per CTA: four (one per TMEM lane quarter, 32 rows x 256 columns each) or eight (two per quarter, 128
// columns each).  Measured in one process at 8192^3 and at 2048 x 8192 x 8192: four are 2 % ahead (350.4 against
// 357.5 us, 94.7 against 96.6 us); the launch runs at the power cap, and warps that only wait still cost.
constexpr int P_EPI_WARPS = 4;
constexpr int P_EPI_BUFS = 1;                       // store buffers (4 KiB) per epilogue warp
constexpr int P_THREADS = 32 * (2 + P_EPI_WARPS);   // 1 TMA warp, 1 MMA warp, the epilogue warps
constexpr int P_WARP_CHUNKS = 8 / (P_EPI_WARPS / 4);   // 32-column chunks of the accumulator one epilogue warp moves
static_assert(P_EPI_WARPS == 4 || P_EPI_WARPS == 8, "one or two epilogue warps per TMEM lane quarter");
struct PairPipeState {
  uint64_t full[P_STAGES];
  uint64_t empty[P_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_word;
  uint32_t peer_abort;     // the peer CTA's abort word, written by the peer before the closing cluster barrier
  uint32_t fills_own;      // ring fills this CTA's producer issued
  uint32_t fills_peer;     // even CTA only: ring fills the odd CTA's producer issued
};

constexpr size_t PAIR_SMEM_BYTES =
    1024 + size_t(P_STAGES) * P_STAGE_BYTES + size_t(P_EPI_WARPS) * P_EPI_BUFS * EPI_BUF_BYTES + 512;
static_assert(PAIR_SMEM_BYTES <= 227 * 1024, "shared memory per CTA");
static_assert(sizeof(PairPipeState) <= 512, "pipeline state outgrew its shared-memory reserve");

// `wait_limit`: cycles a device-side wait may take before the pair gives up (kWaitLimitCycles in production).
// `stop_fill`: test hook, -1 in production; the odd CTA's producer stops before this ring fill as if its wait for the
// stage had run out, so the fill never completes, the even CTA's wait for it runs out and the teardown runs.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
i8gemm_umma_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmC, int M, int N, int K, TileRaster rs,
                        int* __restrict__ status, long long wait_limit, int stop_fill) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = tiles + size_t(P_STAGES) * P_STAGE_BYTES;
  // C is written once and never read here: its lines should be the first to leave L2, so that A and B
  // (128 MiB at 8192^3, about the size of L2) stay (measured +0.5 %).
  const uint64_t store_policy = l2_policy_evict_first();
  PairPipeState* ps = reinterpret_cast<PairPipeState*>(staging + P_EPI_WARPS * P_EPI_BUFS * EPI_BUF_BYTES);
  volatile int* abort_word = &ps->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();          // 0 = even CTA (issues the MMAs), 1 = its peer
  const int pair = blockIdx.x >> 1;

  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = rs.mt * rs.nt;
  const int kblocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&ps->full[s], 1);                    // the even CTA's producer arrives (with both CTAs' bytes)
      mbar_init(&ps->empty[s], 1);                   // one multicast commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&ps->tmem_full[b], 1);               // one multicast commit
      mbar_init(&ps->tmem_empty[b], 2 * P_EPI_WARPS);   // the epilogue warps of both CTAs
    }
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
  // The set-up above may overlap the end of the kernel before this one on the stream; operands, C and the status
  // word are not touched before that kernel has completed.
  grid_dependency_wait();
  grid_launch_dependents();

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t fills = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int mi, ni;
        tile_coords(rs, t, mi, ni);
        const int m0 = mi * 256 + int(rank) * 128, n0 = ni * 256 + int(rank) * 128;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&ps->empty[stage], phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_PRODUCER, wait_limit)) {
            ok = false;
            break;
          }
          if (rank == 1 && int(fills) == stop_fill) {
            atomicCAS(const_cast<int*>(abort_word), 0, KSTAT_WAIT_EXPIRED_PRODUCER);
            ok = false;
            break;
          }
          uint8_t* a_s = tiles + size_t(stage) * P_STAGE_BYTES;
          uint8_t* b_s = a_s + P_A_BYTES;
          if (rank == 0) mbar_arrive_expect_tx(&ps->full[stage], 2 * P_STAGE_BYTES);
          const uint32_t full_even = mapa_shared(smem_u32(&ps->full[stage]), 0);
          tma_load_2d_pair(a_s, &tmA, full_even, kb * BK, m0);
          tma_load_2d_pair(b_s, &tmB, full_even, n0, kb * BK);
          ++fills;
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (ok) {
        // Every stage released => every MMA that reads shared memory has retired before the ring is reused by
        // the last epilogue or given back.
        for (int s = 0; s < P_STAGES; ++s) {
          if (!mbar_wait(&ps->empty[stage], phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_PRODUCER, wait_limit)) break;
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      // How far this producer got, for the teardown of a pair that gave up (see the end of the kernel).
      if (rank == 0) ps->fills_own = fills;
      else st_shared_cluster_u32(mapa_shared(smem_u32(&ps->fills_peer), 0), fills);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA only) ------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_instr_desc(UMMA_D_S32, UMMA_AB_S8, false, true, 256, 256);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        if (!mbar_wait<true>(&ps->tmem_empty[acc], acc_phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_MMA, wait_limit)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + uint32_t(acc * BN);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait<true>(&ps->full[stage], phase, abort_word, KSTAT_WAIT_EXPIRED_MMA, wait_limit)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(tiles + size_t(stage) * P_STAGE_BYTES);
          const uint32_t b_addr = a_addr + P_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t a_desc = umma_smem_desc_sw128(a_addr + kk * UMMA_K, 16, 1024);
            const uint64_t b_desc = umma_smem_desc_sw128(b_addr + kk * UMMA_K * 128, P_B_BYTES, 1024);
            umma_i8<2>(d_tmem, a_desc, b_desc, idesc, uint32_t((kb | kk) != 0));
          }
          umma_commit_pair(&ps->empty[stage], 3);
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair(&ps->tmem_full[acc], 3);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    // Epilogue warp e owns TMEM lane quarter (warp % 4) and, with two warps per quarter, column half (e / 4).
    const int e = warp - 2;
    const int q = warp & 3;
    const int c_begin = (e >> 2) * P_WARP_CHUNKS, c_end = c_begin + P_WARP_CHUNKS;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = pair; t < num_tiles; t += num_pairs) {
      int mi, ni;
      tile_coords(rs, t, mi, ni);
      const int m0 = mi * 256 + int(rank) * 128, n0 = ni * 256;
      const bool ready = mbar_wait<true>(&ps->tmem_full[acc], acc_phase, abort_word, KSTAT_WAIT_EXPIRED_EPILOGUE, wait_limit);
      if (!__all_sync(0xffffffffu, ready)) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * BN);
      // The last tile's epilogue overlaps nothing, and by now every MMA of this pair has read its operands and
      // no load is in flight: the operand ring serves as one store buffer per column chunk (128 KiB in all).
      uint8_t* wide = t + num_pairs < num_tiles ? nullptr : tiles + size_t(e) * P_WARP_CHUNKS * EPI_BUF_BYTES;
      epilogue_warp_tile<P_EPI_BUFS>(t_row, &tmC, staging + e * P_EPI_BUFS * EPI_BUF_BYTES, M, N, m0 + q * 32, n0, lane,
                                     store_policy, wide, c_begin, c_end);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(&ps->tmem_empty[acc], 0);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    // The stores have read their shared-memory buffers; the writes themselves complete before the grid does.
    if (lane == 0) tma_store_wait_read<0>();
    __syncwarp();
  }

  // Neither CTA may free TMEM or leave while its peer's MMAs, commits or remote arrivals can still touch it.
  // The two CTAs also tell each other whether they gave up: a pair that did has to make sure that no copy is
  // still on its way into either CTA's shared memory before the CTAs go.
  tc_fence_before_sync();
  __syncthreads();                                   // every role of this CTA is done: the abort word is final
  if (threadIdx.x == 0)
    st_shared_cluster_u32(mapa_shared(smem_u32(&ps->peer_abort), rank ^ 1u), uint32_t(ps->abort_word));
  cluster_sync_all();
  if (ps->abort_word != 0 || ps->peer_abort != 0) {  // the same verdict in both CTAs
    if (rank == 0 && threadIdx.x == 0 &&
        !pair_drain_loads<P_STAGES>(ps->full, ps->fills_own, ps->fills_peer, P_STAGE_BYTES))
      atomicCAS(&ps->abort_word, 0, KSTAT_WAIT_EXPIRED_DRAIN);
    cluster_sync_all();
  }
  if (warp == 1) tmem_dealloc<2>(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && ps->abort_word != 0) atomicCAS(status, 0, ps->abort_word);
}

}  // namespace

int launch_i8gemm(DeviceCtx* c, const int8_t* A, const int8_t* B, int32_t* C, int64_t M, int64_t N, int64_t K,
                  int raster_mode, int group, int variant, cudaStream_t s, int64_t ldb, int64_t ldc) {
  if (ldb == 0) ldb = N;
  if (ldc == 0) ldc = N;
  if (ldb < N || ldc < N || (ldb & 15) || (ldc & 3)) return fail(VT_ERR_INVALID, "bad row pitch for B or C");
  if (variant == VT_I8_CTA_PAIR_WIDE) return launch_i8gemm_wide(c, A, B, C, M, N, K, raster_mode, group, s, ldb, ldc);
  if (variant != VT_I8_B_AS_STORED && variant != VT_I8_CTA_PAIR)
    return fail(VT_ERR_UNSUPPORTED, "i8gemm variant %d is not built", variant);
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return fail(VT_ERR_INVALID, "i8gemm operands must be 16-byte aligned");
  if (raster_mode < 0 || raster_mode > 2) return fail(VT_ERR_INVALID, "raster mode %d out of range", raster_mode);
  const bool pair = variant != VT_I8_B_AS_STORED;
  const int tile_m = pair ? 256 : BM;

  TileRaster rs;
  rs.mt = int((M + tile_m - 1) / tile_m);
  rs.nt = int((N + BN - 1) / BN);
  rs.mode = raster_mode;
  const int g = pair ? (group + 1) / 2 : group;   // `group` counts 128-row tile-rows
  rs.group = g < 1 ? 1 : (g > rs.mt ? rs.mt : g);
  const long long tiles = 1LL * rs.mt * rs.nt;
  if (tiles > 0x7fffffffLL) return fail(VT_ERR_INVALID, "tile count overflows int");

  CUtensorMap tmA, tmB, tmC;
  int rc = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, uint64_t(K), uint64_t(M), uint64_t(K), BK, 128);
  if (rc) return rc;
  rc = encode_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, C, uint64_t(N), uint64_t(M), uint64_t(ldc) * 4, 32, 32);
  if (rc) return rc;
  rc = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, uint64_t(N), uint64_t(K), uint64_t(ldb), 128, BK);
  if (rc) return rc;
  const int iM = int(M), iN = int(N), iK = int(K);

  if (!pair) {
    const int grid = int(tiles < c->sm_count ? tiles : c->sm_count);
    if (!(c->func_attr_mask & 1u)) {
      VT_CUDA(cudaFuncSetAttribute(i8gemm_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_BYTES)));
      c->func_attr_mask |= 1u;
    }
    VT_CUDA(launch_overlapped(i8gemm_umma_kernel, unsigned(grid), unsigned(NUM_THREADS), SMEM_BYTES, s, tmA, tmB, tmC, iM,
                              iN, iK, rs, c->status));
    count_launch();
    VT_CUDA(cudaGetLastError());
    return VT_OK;
  }
  const int max_pairs = c->sm_count / 2;
  const int pairs = int(tiles < max_pairs ? tiles : max_pairs);
  if (!(c->func_attr_mask & 4u)) {
    VT_CUDA(cudaFuncSetAttribute(i8gemm_umma_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(PAIR_SMEM_BYTES)));
    c->func_attr_mask |= 4u;
  }
  VT_CUDA(launch_overlapped(i8gemm_umma_pair_kernel, unsigned(2 * pairs), unsigned(P_THREADS), PAIR_SMEM_BYTES, s, tmA, tmB,
                            tmC, iM, iN, iK, rs, c->status, c->wait_limit_cycles, c->i8_stop_fill));
  count_launch();
  VT_CUDA(cudaGetLastError());
  return VT_OK;
}

}  // namespace vt
