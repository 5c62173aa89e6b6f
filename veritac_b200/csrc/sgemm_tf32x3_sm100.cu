// fp32 GEMM on the tensor cores by the 3xTF32 split: C = A*B with every fp32 operand written as
// hi + lo, hi = the operand cut to TF32 (its top 19 bits), lo = operand - hi (exact in fp32), and
//     A*B ~= Ahi*Bhi + Alo*Bhi + Ahi*Blo        (the dropped lo*lo term is ~2^-21 relative),
// all three products accumulated in fp32 in one TMEM accumulator by tcgen05.mma.kind::tf32.
// It replaces the same generated `matmul()` loop nest as the FFMA kernel
// (reference specializations/cpu_gemm/emit_c.py:83-155, runner.py:155-190) and is used only where it
// meets the 1e-5 relative-Frobenius contract; the tests hold it to that against float64.
//
// Two kernels:
//   lo_parts_kernel      one streaming pass that writes A lo and B lo.  There are no hi arrays: the
//                        tensor core reads only the top 19 bits of a 32-bit TF32 operand, so A and B
//                        themselves are the hi operands.  HBM-bound (reads and writes 4 bytes per
//                        element of A and B), against several ms of GEMM.
//   sgemm_tf32x3_pair_kernel   the CTA-pair pipeline of the int8 kernel (cta_group::2, 256x256 tile per
//                        pair, TMA-staged swizzled operands, double-buffered TMEM accumulator,
//                        TMA-store epilogue) with BK = 32 floats, four operand tiles per stage (A,
//                        A lo: K-major, 128-byte swizzle; B, B lo: as stored, N contiguous, which for
//                        32-bit operands needs the "128 B swizzle with 32 B atoms" layout; 64 KiB per
//                        CTA, 3 stages) and three MMAs per K step of 8.
#include "ptx_sm100.cuh"
#include "runtime.h"
#include "umma_tile.cuh"

namespace vt {
namespace {

constexpr int T_BK = 32;                       // floats per K block = one 128-byte swizzle row
constexpr int T_UMMA_K = 8;                    // tf32 MMA depth
constexpr int T_STAGES = 3;
constexpr int T_CHUNK_KB = 4;                   // K blocks (of 32) folded into one TMEM accumulator
constexpr int T_THREADS = 384;                 // warpgroup 0: TMA warp, MMA warp, 2 idle; warpgroups 1-2: 8 epilogue warps
constexpr int T_A_BYTES = 128 * T_BK * 4;      // 128 rows x 128 B = 16 KiB (hi or lo)
constexpr int T_B_BYTES = 128 * T_BK * 4;      // this CTA's 128 columns of B for 32 rows of K (B or B lo)
constexpr int T_B_BOX_BYTES = 32 * T_BK * 4;   // one TMA box: 32 columns x 32 rows
constexpr int T_STAGE_BYTES = 2 * T_A_BYTES + 2 * T_B_BYTES;   // 64 KiB

struct TfPipeState {
  uint64_t full[T_STAGES];
  uint64_t empty[T_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_word;
  uint32_t peer_abort;     // the peer CTA's abort word, written by the peer before the closing cluster barrier
  uint32_t fills_own;      // ring fills this CTA's producer issued
  uint32_t fills_peer;     // even CTA only: ring fills the odd CTA's producer issued
};

constexpr size_t T_SMEM_BYTES = 1024 + size_t(T_STAGES) * T_STAGE_BYTES + EPI_STAGING_BYTES + sizeof(TfPipeState);

// lo parts of A and of B in one streaming pass: lo = x - (x cut to its top 19 bits), exact, with half
// of its own cut-off unit added to the bit pattern so that the tensor core's cut rounds it to nearest.
// The hi parts need no pass: the tensor core reads the top 19 bits of the operands as they are.
__device__ __forceinline__ float tf32_lo_part(float x) {
  const float hi = __uint_as_float(__float_as_uint(x) & 0xffffe000u);
  return __uint_as_float(__float_as_uint(x - hi) + 0x1000u);
}
__global__ void __launch_bounds__(256) lo_parts_kernel(const float4* __restrict__ a, float4* __restrict__ a_lo, int64_t na4,
                                                      const float4* __restrict__ b, float4* __restrict__ b_lo, int64_t nb4) {
  // Launched for overlap with the kernel before it (see launch_overlapped): the lo parts overwrite scratch that
  // a product still running may be reading, so nothing is touched before that kernel has completed.
  grid_dependency_wait();
  grid_launch_dependents();
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < na4 + nb4; i += stride) {
    const bool in_a = i < na4;
    const float4 v = __ldcs(in_a ? a + i : b + (i - na4));
    const float4 l = make_float4(tf32_lo_part(v.x), tf32_lo_part(v.y), tf32_lo_part(v.z), tf32_lo_part(v.w));
    if (in_a) a_lo[i] = l;
    else b_lo[i - na4] = l;
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T_THREADS, 1)
sgemm_tf32x3_pair_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
                         const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl,
                         const __grid_constant__ CUtensorMap tmC, int M, int N, int K, TileRaster rs,
                         int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = tiles + size_t(T_STAGES) * T_STAGE_BYTES;
  TfPipeState* ps = reinterpret_cast<TfPipeState*>(staging + EPI_STAGING_BYTES);
  volatile int* abort_word = &ps->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = rs.mt * rs.nt;
  const int kblocks = (K + T_BK - 1) / T_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T_STAGES; ++s) {
      mbar_init(&ps->full[s], 1);
      mbar_init(&ps->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&ps->tmem_full[b], 1);
      mbar_init(&ps->tmem_empty[b], 16);   // 8 epilogue warps of each CTA
    }
    ps->abort_word = 0;
    ps->peer_abort = 0;
    ps->fills_own = 0;
    ps->fills_peer = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmAh);
    tma_prefetch_desc(&tmAl);
    tma_prefetch_desc(&tmBh);
    tma_prefetch_desc(&tmBl);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc<2>(&ps->tmem_base, TMEM_COLS);
    tmem_relinquish<2>();
  }
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = ps->tmem_base;
  // The set-up above may overlap the end of the lo-part pass (or of whatever kernel precedes this one on the
  // stream); operands, lo parts, C and the status word are not touched before it has completed.
  grid_dependency_wait();
  grid_launch_dependents();

  // Register budget by warpgroup: the epilogue keeps 128 fp32 partial sums per thread, the
  // producer and MMA threads need almost nothing.  (40 + 232 + 232) * 128 <= 65536.
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
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
          if (!mbar_wait(&ps->empty[stage], phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_PRODUCER)) {
            ok = false;
            break;
          }
          uint8_t* a_hi = tiles + size_t(stage) * T_STAGE_BYTES;
          uint8_t* a_lo = a_hi + T_A_BYTES;
          uint8_t* b_hi = a_lo + T_A_BYTES;
          uint8_t* b_lo = b_hi + T_B_BYTES;
          if (rank == 0) mbar_arrive_expect_tx(&ps->full[stage], 2 * T_STAGE_BYTES);
          const uint32_t full_even = mapa_shared(smem_u32(&ps->full[stage]), 0);
          const int k0 = kb * T_BK;
          tma_load_2d_pair(a_hi, &tmAh, full_even, k0, m0);
          tma_load_2d_pair(a_lo, &tmAl, full_even, k0, m0);
#pragma unroll
          for (int b = 0; b < 4; ++b) {   // this CTA's 128 columns of B as stored: four boxes of 32 columns x 32 rows
            tma_load_2d_pair(b_hi + b * T_B_BOX_BYTES, &tmBh, full_even, n0 + 32 * b, k0);
            tma_load_2d_pair(b_lo + b * T_B_BOX_BYTES, &tmBl, full_even, n0 + 32 * b, k0);
          }
          ++fills;
          if (++stage == T_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (ok) {
        for (int s = 0; s < T_STAGES; ++s) {
          if (!mbar_wait(&ps->empty[stage], phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_PRODUCER)) break;
          if (++stage == T_STAGES) {
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
    // The tensor core adds into its fp32 accumulator with truncation, so the error of one
    // accumulator grows linearly with the number of K steps folded into it (measured 7e-9 * K
    // relative).  Each accumulator therefore takes only T_CHUNK_KB K blocks (128 values of K);
    // the epilogue warps add finished chunks into fp32 registers with round-to-nearest while the
    // next chunk runs in the other accumulator.
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_instr_desc(UMMA_D_F32, UMMA_AB_TF32, false, true, 256, 256);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        for (int kb0 = 0; kb0 < kblocks && ok; kb0 += T_CHUNK_KB) {
          if (!mbar_wait<true>(&ps->tmem_empty[acc], acc_phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + uint32_t(acc * BN);
          const int kb1 = min(kblocks, kb0 + T_CHUNK_KB);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait<true>(&ps->full[stage], phase, abort_word, KSTAT_WAIT_EXPIRED_MMA)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t a_hi = smem_u32(tiles + size_t(stage) * T_STAGE_BYTES);
            const uint32_t a_lo = a_hi + T_A_BYTES;
            const uint32_t b_hi = a_lo + T_A_BYTES;
            const uint32_t b_lo = b_hi + T_B_BYTES;
#pragma unroll
            for (int kk = 0; kk < T_BK / T_UMMA_K; ++kk) {
              // A tiles are K-major: 8 floats = 32 bytes per K step inside the swizzle row.  B tiles
              // are B as stored (N contiguous): a K step of 8 rows moves 1 KiB.
              const uint64_t ah = umma_smem_desc_sw128(a_hi + kk * 32, 16, 1024);
              const uint64_t al = umma_smem_desc_sw128(a_lo + kk * 32, 16, 1024);
              const uint64_t bh = umma_smem_desc_mn32(b_hi + kk * 1024, T_B_BOX_BYTES);
              const uint64_t bl = umma_smem_desc_mn32(b_lo + kk * 1024, T_B_BOX_BYTES);
              // small terms first, the dominant product last
              umma_tf32<2>(d_tmem, al, bh, idesc, uint32_t((kb != kb0) || kk != 0));
              umma_tf32<2>(d_tmem, ah, bl, idesc, 1u);
              umma_tf32<2>(d_tmem, ah, bh, idesc, 1u);
            }
            umma_commit_pair(&ps->empty[stage], 3);
            if (++stage == T_STAGES) {
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
    }
    __syncwarp();
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;" ::: "memory");
    // ------------------------------ epilogue (both CTAs, 8 warps) ------------------------------
    // Warp e of 8 owns TMEM lane quarter (warp % 4) and column half (e / 4): 32 rows x 128 columns,
    // one row per thread, kept as 128 fp32 registers for the whole K loop.
    const int e = warp - 4;
    const int q = warp & 3;
    const int half = e >> 2;
    uint8_t* stage_buf = staging + e * EPI_BUF_BYTES;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool alive = true;
    for (int t = pair; t < num_tiles && alive; t += num_pairs) {
      int mi, ni;
      tile_coords(rs, t, mi, ni);
      const int row0 = mi * 256 + int(rank) * 128 + q * 32;
      const int col0 = ni * 256 + half * 128;
      float master[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) master[i] = 0.f;
      for (int kb0 = 0; kb0 < kblocks; kb0 += T_CHUNK_KB) {
        const bool ready = mbar_wait<true>(&ps->tmem_full[acc], acc_phase, abort_word, KSTAT_WAIT_EXPIRED_EPILOGUE);
        if (!__all_sync(0xffffffffu, ready)) {
          alive = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * BN + half * 128);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(t_row + uint32_t(c * 16), r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) master[c * 16 + i] += __uint_as_float(r[i]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(&ps->tmem_empty[acc], 0);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
      if (!alive) break;
      // registers -> swizzled shared memory -> TMA store, 32 columns at a time.  After the pair's last tile every
      // MMA has read its operands and no load is in flight: the idle operand ring then gives each chunk a buffer
      // of its own (8 warps x 4 x 4 KiB) and no store waits for the one before it.
      const bool last = t + num_pairs >= num_tiles;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint8_t* buf = last ? tiles + size_t(e * 4 + c) * EPI_BUF_BYTES : stage_buf;
        if (!last) {
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
        }
        const uint32_t base = smem_u32(buf) + uint32_t(lane) * 128u;
#pragma unroll
        for (int v = 0; v < 8; ++v)
          st_shared_v4(base + (uint32_t(v ^ (lane & 7)) << 4), __float_as_uint(master[c * 32 + 4 * v]),
                       __float_as_uint(master[c * 32 + 4 * v + 1]), __float_as_uint(master[c * 32 + 4 * v + 2]),
                       __float_as_uint(master[c * 32 + 4 * v + 3]));
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (row0 < M && col0 + c * 32 < N) tma_store_2d(&tmC, buf, col0 + c * 32, row0);
          tma_store_commit();
        }
      }
    }
    // The stores have read their shared-memory buffers; the writes themselves complete before the grid does.
    if (lane == 0) tma_store_wait_read<0>();
    __syncwarp();
  }

  // Neither CTA may free TMEM or leave while its peer's MMAs, commits or remote arrivals can still touch it.
  // The two CTAs also tell each other whether they gave up: a pair that did makes sure that no copy is still on
  // its way into either CTA's shared memory before the CTAs go (pair_drain_loads, umma_tile.cuh).
  tc_fence_before_sync();
  __syncthreads();                                   // every role of this CTA is done: the abort word is final
  if (threadIdx.x == 0)
    st_shared_cluster_u32(mapa_shared(smem_u32(&ps->peer_abort), rank ^ 1u), uint32_t(ps->abort_word));
  cluster_sync_all();
  if (ps->abort_word != 0 || ps->peer_abort != 0) {  // the same verdict in both CTAs
    if (rank == 0 && threadIdx.x == 0 &&
        !pair_drain_loads<T_STAGES>(ps->full, ps->fills_own, ps->fills_peer, T_STAGE_BYTES))
      atomicCAS(&ps->abort_word, 0, KSTAT_WAIT_EXPIRED_DRAIN);
    cluster_sync_all();
  }
  if (warp == 1) tmem_dealloc<2>(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && ps->abort_word != 0) atomicCAS(status, 0, ps->abort_word);
}


}  // namespace

bool sgemm_tf32x3_supported(const float* A, const float* B, const float* C, int64_t M, int64_t N, int64_t K) {
  (void)M;
  return N % 4 == 0 && K % 4 == 0 &&
         ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) == 0;
}

size_t sgemm_tf32x3_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  return (size_t(M) * K + size_t(K) * N) * sizeof(float);
}

// `split` holds B lo | A lo back to back (sgemm_tf32x3_workspace_bytes); B lo comes first so that callers
// who feed A in row blocks against one B keep B lo where it is.
//   parts: 1 = write A lo, 2 = write B lo, 3 = both (the whole product in one call)
int launch_sgemm_tf32x3(DeviceCtx* c, const float* A, const float* B, float* C, float* split, int64_t M, int64_t N,
                        int64_t K, cudaStream_t s, int parts) {
  if (!sgemm_tf32x3_supported(A, B, C, M, N, K))
    return fail(VT_ERR_UNSUPPORTED, "3xTF32 kernel needs N %% 4 == 0, K %% 4 == 0 and 16-byte aligned operands");
  const size_t na = size_t(M) * K, nb = size_t(K) * N;
  float* Bl = split;
  float* Al = Bl + nb;
  if (parts & 3) {
    const int blocks = c->sm_count * 8;
    VT_CUDA(launch_overlapped(lo_parts_kernel, unsigned(blocks), 256u, size_t(0), s, reinterpret_cast<const float4*>(A),
                              reinterpret_cast<float4*>(Al), (parts & 1) ? int64_t(na / 4) : int64_t(0),
                              reinterpret_cast<const float4*>(B), reinterpret_cast<float4*>(Bl),
                              (parts & 2) ? int64_t(nb / 4) : int64_t(0)));
    count_launch();
  }
  if (M == 0) return VT_OK;   // B lo only

  TileRaster rs;
  rs.mt = int((M + 255) / 256);
  rs.nt = int((N + 255) / 256);
  rs.mode = 2;
  rs.group = rs.mt < 8 ? rs.mt : 8;
  const long long tiles = 1LL * rs.mt * rs.nt;
  if (tiles > 0x7fffffffLL) return fail(VT_ERR_INVALID, "tile count overflows int");
  CUtensorMap tmAh, tmAl, tmBh, tmBl, tmC;
  int rc = 0;
  const CUtensorMapDataType f32 = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const CUtensorMapSwizzle mn32 = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
  if ((rc = encode_tmap_2d(&tmAh, f32, 4, A, uint64_t(K), uint64_t(M), uint64_t(K) * 4, T_BK, 128))) return rc;
  if ((rc = encode_tmap_2d(&tmAl, f32, 4, Al, uint64_t(K), uint64_t(M), uint64_t(K) * 4, T_BK, 128))) return rc;
  if ((rc = encode_tmap_2d(&tmBh, f32, 4, B, uint64_t(N), uint64_t(K), uint64_t(N) * 4, 32, T_BK, mn32))) return rc;
  if ((rc = encode_tmap_2d(&tmBl, f32, 4, Bl, uint64_t(N), uint64_t(K), uint64_t(N) * 4, 32, T_BK, mn32))) return rc;
  if ((rc = encode_tmap_2d(&tmC, f32, 4, C, uint64_t(N), uint64_t(M), uint64_t(N) * 4, 32, 32))) return rc;
  if (!(c->func_attr_mask & 32u)) {
    VT_CUDA(cudaFuncSetAttribute(sgemm_tf32x3_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(T_SMEM_BYTES)));
    c->func_attr_mask |= 32u;
  }
  const int max_pairs = c->sm_count / 2;
  const int pairs = int(tiles < max_pairs ? tiles : max_pairs);
  VT_CUDA(launch_overlapped(sgemm_tf32x3_pair_kernel, unsigned(2 * pairs), unsigned(T_THREADS), size_t(T_SMEM_BYTES), s,
                            tmAh, tmAl, tmBh, tmBl, tmC, int(M), int(N), int(K), rs, c->status));
  count_launch();
  VT_CUDA(cudaGetLastError());
  return VT_OK;
}

}  // namespace vt
