// Pieces shared by the tcgen05 GEMM kernels (int8 and 3xTF32): tile order, the TMEM -> C epilogue
// of one warp, and the constants both pipelines agree on.  Accumulator tiles are 128 lanes x 256
// 32-bit columns per CTA whatever the operand type.
#pragma once

#include "ptx_sm100.cuh"

namespace vt {
namespace {

constexpr int BN = 256;                             // accumulator columns per tile
constexpr int NUM_THREADS = 192;                    // 1 TMA warp, 1 MMA warp, 4 epilogue warps
constexpr int TMEM_COLS = 512;                      // two 256-column 32-bit accumulators

// Epilogue staging: each epilogue warp owns one or two 32-row x 32-column int32 buffers (4 KiB each,
// 128-byte rows in the 128-byte swizzle the C tensor map expects).
constexpr int EPI_BUF_BYTES = 32 * 32 * 4;
constexpr int EPI_STAGING_BYTES = 4 * 2 * EPI_BUF_BYTES;   // 32 KiB

struct TileRaster {
  int mt, nt;  // tile counts along M and N
  int mode;    // 0 row-major, 1 column-major, 2 grouped
  int group;   // tile-rows per column sweep (mode 2)
};

__device__ __forceinline__ void tile_coords(const TileRaster& rs, int t, int& mi, int& ni) {
  if (rs.mode == 0) {
    mi = t / rs.nt;
    ni = t - mi * rs.nt;
  } else if (rs.mode == 1) {
    ni = t / rs.mt;
    mi = t - ni * rs.mt;
  } else {
    const int per = rs.group * rs.nt;
    const int g = t / per;
    const int w = t - g * per;
    const int rows = min(rs.group, rs.mt - g * rs.group);
    ni = w / rows;
    mi = g * rs.group + (w - ni * rows);
  }
}

// Moves one warp's 32 rows x 32 (c_end - c_begin) columns of an accumulator from TMEM to C: TMEM -> registers ->
// swizzled shared memory -> cp.async.bulk.tensor store, so C is written in whole 128-byte lines and
// rows/columns outside C are clipped by the TMA unit.
// `wide`, when given, is one further buffer per column chunk (4 KiB each, 1024-byte aligned) that nothing else uses any more: every
// column chunk then gets a buffer of its own and no store waits for the one before it (the last tile of a
// CTA, whose epilogue nothing overlaps, takes them from the idle operand ring).
// A `wide` area of fewer buffers than chunks (kWide) is used round-robin: a chunk then waits for the store that
// last read its buffer.
// Returns once the accumulator has been read (the stores may still be in flight).
template <int kBufs = 2, int kWide = 16>
__device__ __forceinline__ void epilogue_warp_tile(uint32_t t_row, const CUtensorMap* tmC, uint8_t* staging, int M,
                                                   int N, int row0, int n0, int lane, uint64_t store_policy = 0,
                                                   uint8_t* wide = nullptr, int c_begin = 0, int c_end = BN / 32) {
#pragma unroll 1
  for (int c = c_begin; c < c_end; ++c) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(t_row + uint32_t(c * 32), r);
    tmem_ld_wait();
    uint8_t* buf = wide ? wide + ((c - c_begin) % kWide) * EPI_BUF_BYTES : staging + (c & (kBufs - 1)) * EPI_BUF_BYTES;
    if (!wide) {
      if (lane == 0) tma_store_wait_read<kBufs - 1>();   // the store that last read this buffer is done with it
      __syncwarp();
    } else if (c - c_begin >= kWide) {
      if (lane == 0) tma_store_wait_read<kWide - 1>();
      __syncwarp();
    }
    const uint32_t base = smem_u32(buf) + uint32_t(lane) * 128u;
#pragma unroll
    for (int v = 0; v < 8; ++v)
      st_shared_v4(base + (uint32_t(v ^ (lane & 7)) << 4), r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (row0 < M && n0 + c * 32 < N) {
        if (store_policy) tma_store_2d_hint(tmC, buf, n0 + c * 32, row0, store_policy);
        else tma_store_2d(tmC, buf, n0 + c * 32, row0);
      }
      tma_store_commit();
    }
  }
}

// Teardown of a CTA pair whose pipeline gave up, run by one thread of the even CTA after both CTAs have stopped
// issuing copies.  Both CTAs' operand copies are counted on the even CTA's `full` barriers, which its producer
// arms for the two of them; `fills_even` / `fills_odd` say how many ring fills each producer got to.  A fill
// that only one of them reached can never complete by itself, so the books are balanced first (bytes that will
// never come are written off; a copy of the peer that was never armed is armed now), and then the last fill of
// every stage is waited for, with a limit.  After this no copy is in flight into either CTA's shared memory.
template <int kStages>
__device__ __forceinline__ bool pair_drain_loads(uint64_t* full, uint32_t fills_even, uint32_t fills_odd,
                                                 uint32_t bytes_per_cta) {
  const uint32_t hi = fills_even > fills_odd ? fills_even : fills_odd;
  uint32_t lo = fills_even > fills_odd ? fills_odd : fills_even;
  if (hi - lo > uint32_t(kStages)) lo = hi - uint32_t(kStages);
  for (uint32_t f = lo; f < hi; ++f) {
    uint64_t* bar = &full[f % uint32_t(kStages)];
    if (fills_even > fills_odd) mbar_complete_tx(bar, bytes_per_cta);
    else mbar_arrive_expect_tx(bar, bytes_per_cta);
  }
  bool ok = true;
  for (uint32_t f = hi > uint32_t(kStages) ? hi - uint32_t(kStages) : 0; f < hi; ++f)
    ok = mbar_wait_drain(&full[f % uint32_t(kStages)], (f / uint32_t(kStages)) & 1u) && ok;
  return ok;
}

}  // namespace
}  // namespace vt
