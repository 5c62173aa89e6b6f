// Skinny fp32 GEMM (M <= 16) as one HBM-bound stream of B: TMA-fed, products on the tensor cores,
// one launch.
//
//   grid      exactly (resident CTAs per SM) x (SM count) CTAs, all running from the first cycle to
//             the last: no second wave and no tail of late CTAs, whose few copies in flight could
//             not keep HBM busy.  B is cut into 128-column slabs and 32-row chunks.  With G CTAs
//             and S slabs, floor(G/S) "regular" CTAs per slab split the upper rows of the slab
//             evenly (CTA c -> slab c mod S, so neighbours read neighbouring 512-byte segments of
//             the same rows); the G mod S CTAs left over share the bottom rows of all slabs in
//             equal pieces, a piece running on from one slab into the next.  The row where the
//             bottom part starts is chosen so that every CTA gets the same number of chunks.
//   loads     one elected thread issues four 32x32 TMA boxes (128-byte swizzle) per 32-row chunk into
//             a 4-stage ring; full/empty mbarriers, no CTA-wide barrier in the main loop.
//   math      each of 4 warps owns 32 columns: 16x8x8 TF32 mma.sync with every operand split into
//             hi + lo in registers (three MMAs per product, small terms first), accumulators
//             folded into fp32 registers after every chunk so the tensor core's truncating
//             accumulation never runs over more than 32 values of K.  M = 16 is the MMA's M.
//             A's fragments come straight from global memory (L1/L2 resident: A is M x K).
//             The MMA's k slots map to rows (0,2,4,6 | 1,3,5,7) of each 8-row step, which makes
//             the swizzled B fragment loads bank-conflict free.
//   K split   a slab's CTAs leave partial tiles in scratch memory; the CTA that finishes last
//             (a ticket per slab) sums them in split order and writes C, so results do not depend
//             on which CTA that is.  Tickets return to zero for the next launch.
#include <cstdlib>
#include "ptx_sm100.cuh"
#include "runtime.h"
#include "skinny_sched.cuh"

namespace vt {
namespace {

constexpr int KT_COLS = SKINNY_COLS;
constexpr int KT_KC = SKINNY_KC;
constexpr int KT_STAGES = 4;
constexpr int KT_CONSUMERS = 4;              // warps
constexpr int KT_THREADS = 32 * (KT_CONSUMERS + 1);
constexpr int KT_BOX_BYTES = 32 * 32 * 4;    // one TMA box: 32 rows x 32 floats
constexpr int KT_STAGE_BYTES = 4 * KT_BOX_BYTES;
constexpr int KT_CTAS_PER_SM = 3;
constexpr int KT_PIECE_OVERHEAD = 3;         // chunks' worth of time between two pieces of work
constexpr int KT_FOLD = 2;                   // chunks per run of tensor-core accumulation (64 values of K)
constexpr size_t KT_SMEM_BYTES = 1024 + size_t(KT_STAGES) * KT_STAGE_BYTES + 128;

struct SkinnyPipe {
  uint64_t full[KT_STAGES];
  uint64_t empty[KT_STAGES];
  int abort_word;
  int last_flag;
};

__device__ __forceinline__ void mma_16x8x8_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool kVecA>
__global__ void __launch_bounds__(KT_THREADS, KT_CTAS_PER_SM)
sgemm_skinny_tma_kernel(const __grid_constant__ CUtensorMap tmB, const float* __restrict__ A,
                        float* __restrict__ C, float* __restrict__ partials, int* __restrict__ tickets, int M, int N,
                        int K, SkinnySched sc, int* __restrict__ status) {
  extern __shared__ uint8_t kt_smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(kt_smem_raw) + 1023) & ~uintptr_t(1023));
  SkinnyPipe* ps = reinterpret_cast<SkinnyPipe*>(tiles + size_t(KT_STAGES) * KT_STAGE_BYTES);
  volatile int* abort_word = &ps->abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = int(blockIdx.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < KT_STAGES; ++s) {
      mbar_init(&ps->full[s], 1);
      mbar_init(&ps->empty[s], KT_CONSUMERS);
    }
    ps->abort_word = 0;
    ps->last_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();

  if (warp == KT_CONSUMERS) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmB);
      uint32_t filled = 0, fill_parity = 0;
      int it = 0;   // chunks issued by this CTA so far: position in the ring
      bool ok = true;
      SkinnySegment seg;
      for (int idx = 0; ok && sched_segment(sc, cta, idx, seg); ++idx) {
        const int n0 = seg.slab * KT_COLS;
        for (int ch = seg.chunk_beg; ch < seg.chunk_end; ++ch, ++it) {
          const int stage = it % KT_STAGES;
          const uint32_t phase = uint32_t(it / KT_STAGES) & 1u;
          if (it >= KT_STAGES && !mbar_wait(&ps->empty[stage], phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_PRODUCER)) {
            ok = false;
            break;
          }
          uint64_t* full = &ps->full[stage];
          uint8_t* dst = tiles + size_t(stage) * KT_STAGE_BYTES;
          mbar_arrive_expect_tx(full, KT_STAGE_BYTES);
#pragma unroll
          for (int b = 0; b < 4; ++b) tma_load_2d(dst + b * KT_BOX_BYTES, &tmB, full, n0 + 32 * b, ch * KT_KC);
          filled |= 1u << stage;
          fill_parity = (fill_parity & ~(1u << stage)) | (phase << stage);
        }
      }
      if (*abort_word != 0) {
        // Aborting: wait (bounded) for the copies already issued before shared memory goes back.
        for (int s = 0; s < KT_STAGES; ++s)
          if (filled & (1u << s)) mbar_wait_drain(&ps->full[s], (fill_parity >> s) & 1u);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ consumers ------------------------------
    const int g = lane >> 2, t = lane & 3;
    float master[4][4];   // [n-tile][c0..c3]: rows g / g+8, columns 2t / 2t+1 of the n-tile
    float acc[4][4];      // tensor-core accumulators, folded into master every KT_FOLD chunks

    // A fragments of one chunk: for each 8-row step, rows g and g+8 at k = 2t and 2t+1 (adjacent:
    // one 8-byte load when A's rows are 8-byte aligned).
    const bool row_lo = g < M, row_hi = g + 8 < M;
    const float* a_lo = A + size_t(row_lo ? g : 0) * size_t(K);
    const float* a_hi = A + size_t(row_hi ? g + 8 : 0) * size_t(K);
    auto load_a = [&](int chunk, float (&v)[16]) {
      const int k0 = chunk * KT_KC + 2 * t;
#pragma unroll
      for (int ks = 0; ks < KT_KC / 8; ++ks) {
        const int k = k0 + ks * 8;
        if constexpr (kVecA) {
          const bool in = k < K;   // K is even here, so k + 1 < K as well
          const float2 lo = (row_lo && in) ? __ldg(reinterpret_cast<const float2*>(a_lo + k)) : make_float2(0.f, 0.f);
          const float2 hi = (row_hi && in) ? __ldg(reinterpret_cast<const float2*>(a_hi + k)) : make_float2(0.f, 0.f);
          v[4 * ks + 0] = lo.x;
          v[4 * ks + 1] = hi.x;
          v[4 * ks + 2] = lo.y;
          v[4 * ks + 3] = hi.y;
        } else {
          const bool in0 = k < K, in1 = k + 1 < K;
          v[4 * ks + 0] = (row_lo && in0) ? __ldg(a_lo + k) : 0.f;
          v[4 * ks + 1] = (row_hi && in0) ? __ldg(a_hi + k) : 0.f;
          v[4 * ks + 2] = (row_lo && in1) ? __ldg(a_lo + k + 1) : 0.f;
          v[4 * ks + 3] = (row_hi && in1) ? __ldg(a_hi + k + 1) : 0.f;
        }
      }
    };
    // hi = the value rounded to TF32's 10 mantissa bits (half away from zero, in integer arithmetic
    // on the bit pattern), lo = the exact rest; the tensor core reads lo's top bits.
    // The rounding must not carry a finite value into infinity, and an infinity or NaN has no lo part
    // (inf - inf would turn every product of the row into NaN).
    auto split = [](float x, uint32_t& hi, uint32_t& lo) {
      const uint32_t bits = __float_as_uint(x);
      uint32_t h = (bits + 0x1000u) & 0xffffe000u;
      if ((h & 0x7f800000u) == 0x7f800000u) h = bits & 0xffffe000u;
      const float rest = x - __uint_as_float(h);
      hi = h;
      lo = rest == rest ? __float_as_uint(rest) : 0u;
    };
    // Lane-constant offsets of this lane's B elements inside a box, per n-tile.
    int off0[4], off1[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int unit = 2 * j + (g >> 2);
      off0[j] = (2 * t) * 32 + ((unit ^ (2 * t)) << 2) + (g & 3);
      off1[j] = (2 * t + 1) * 32 + ((unit ^ (2 * t + 1)) << 2) + (g & 3);
    }
    auto compute = [&](int stage, const float (&a)[16]) {
      // This warp's box: 32 rows of 128 bytes, 16-byte units XOR-swizzled with (row % 8).
      const float* box = reinterpret_cast<const float*>(tiles + size_t(stage) * KT_STAGE_BYTES + warp * KT_BOX_BYTES);
#pragma unroll
      for (int ks = 0; ks < KT_KC / 8; ++ks) {
        uint32_t fh[4], fl[4], bh0[4], bh1[4], bl0[4], bl1[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) split(a[4 * ks + e], fh[e], fl[e]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          split(box[ks * 256 + off0[j]], bh0[j], bl0[j]);
          split(box[ks * 256 + off1[j]], bh1[j], bl1[j]);
        }
        // Small terms first; the four n-tiles alternate so that no MMA waits on the one before it.
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_16x8x8_tf32(acc[j], fl, bh0[j], bh1[j]);
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_16x8x8_tf32(acc[j], fh, bl0[j], bl1[j]);
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_16x8x8_tf32(acc[j], fh, bh0[j], bh1[j]);
      }
    };
    auto fold = [&]() {
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          master[j][e] += acc[j][e];
          acc[j][e] = 0.f;
        }
    };

    int it = 0;   // chunks consumed by this CTA so far: position in the ring
    bool ok = true;
    SkinnySegment seg;
    for (int idx = 0; sched_segment(sc, cta, idx, seg); ++idx) {
      const int n0 = seg.slab * KT_COLS;
      const int nchunks = seg.chunk_end - seg.chunk_beg;
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) master[j][e] = acc[j][e] = 0.f;

      float a_even[16], a_odd[16];
      if (nchunks > 0) load_a(seg.chunk_beg, a_even);
      for (int i = 0; i < nchunks && ok; i += 2) {
        const int stage0 = it % KT_STAGES, stage1 = (it + 1) % KT_STAGES;
        const uint32_t phase0 = uint32_t(it / KT_STAGES) & 1u, phase1 = uint32_t((it + 1) / KT_STAGES) & 1u;
        if (i + 1 < nchunks) load_a(seg.chunk_beg + i + 1, a_odd);
        // every lane polls; the vote brings the warp back together before the warp-wide MMAs below
        ok = __all_sync(0xffffffffu, mbar_wait(&ps->full[stage0], phase0, abort_word, KSTAT_WAIT_EXPIRED_MMA));
        if (!ok) break;
        compute(stage0, a_even);
        __syncwarp();
        if (lane == 0) mbar_arrive(&ps->empty[stage0]);
        ++it;
        if (i + 1 < nchunks) {
          if (i + 2 < nchunks) load_a(seg.chunk_beg + i + 2, a_even);
          ok = __all_sync(0xffffffffu, mbar_wait(&ps->full[stage1], phase1, abort_word, KSTAT_WAIT_EXPIRED_MMA));
          if (!ok) break;
          compute(stage1, a_odd);
          __syncwarp();
          if (lane == 0) mbar_arrive(&ps->empty[stage1]);
          ++it;
        }
        if (KT_FOLD == 2 || (i & (KT_FOLD - 1)) == KT_FOLD - 2) fold();
      }
      fold();

      // Whether the CTA is giving up is read after a barrier of the four consumer warps, where none
      // of them can still be in a wait, so all of them take the same way out.
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*abort_word != 0) break;
      // The tile of this piece goes to C (the slab has one piece) or to its slot among the slab's partial tiles.
      float* dst = seg.parts == 1 ? C : partials + size_t(seg.part) * size_t(M) * size_t(N);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = n0 + warp * 32 + j * 8 + 2 * t;   // N % 4 == 0 and col even: the pair is in or out together
        if (col < N) {
          if (row_lo) *reinterpret_cast<float2*>(dst + size_t(g) * N + col) = make_float2(master[j][0], master[j][1]);
          if (row_hi)
            *reinterpret_cast<float2*>(dst + size_t(g + 8) * N + col) = make_float2(master[j][2], master[j][3]);
        }
      }
      if (seg.parts > 1)
        skinny_finish_piece<128>(seg, int(threadIdx.x), 1, &ps->last_flag, tickets, partials, C, M, N);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && ps->abort_word != 0) atomicCAS(status, 0, ps->abort_word);
}

}  // namespace

// CTAs in the grid, slabs, and the largest number of partial tiles any slab has (1 = no scratch).
void sgemm_skinny_tma_plan(int64_t N, int64_t K, int sm_count, int* ctas, int* slabs, int* max_parts) {
  const SkinnySched sc = make_skinny_sched(N, K, sm_count, KT_CTAS_PER_SM, KT_PIECE_OVERHEAD, ctas);
  *slabs = sc.slabs;
  *max_parts = skinny_max_parts(sc);
}

bool sgemm_skinny_tma_supported(const float* B, const float* C, int64_t M, int64_t N, int64_t K) {
  return M >= 1 && M <= 16 && N % 4 == 0 && N >= 4 && N <= int64_t(kTicketCount) * SKINNY_COLS && K >= 1 && K < (1LL << 31) &&
         ((reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) == 0;
}

int launch_sgemm_skinny_tma(DeviceCtx* c, const float* A, const float* B, float* C, float* partials, int* tickets,
                            int64_t M, int64_t N, int64_t K, cudaStream_t s) {
  if (!sgemm_skinny_tma_supported(B, C, M, N, K))
    return fail(VT_ERR_UNSUPPORTED, "skinny TMA kernel needs M <= 16, N %% 4 == 0 and 16-byte aligned B and C");
  int ctas, slabs, max_parts;
  sgemm_skinny_tma_plan(N, K, c->sm_count, &ctas, &slabs, &max_parts);
  const SkinnySched sc = make_skinny_sched(N, K, c->sm_count, KT_CTAS_PER_SM, KT_PIECE_OVERHEAD, &ctas);
  if (max_parts > 1 && (!partials || !tickets)) return fail(VT_ERR_INVALID, "skinny K split needs scratch memory");
  if (slabs > kTicketCount)
    return fail(VT_ERR_UNSUPPORTED, "N = %lld has more slabs than the library keeps tickets for", (long long)N);
  CUtensorMap tmB;
  int rc = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, B, uint64_t(N), uint64_t(K), uint64_t(N) * 4, 32, 32);
  if (rc) return rc;
  constexpr uint32_t attr_bit = 1u << 20;
  if (!(c->func_attr_mask & attr_bit)) {
    VT_CUDA(cudaFuncSetAttribute(sgemm_skinny_tma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(KT_SMEM_BYTES)));
    VT_CUDA(cudaFuncSetAttribute(sgemm_skinny_tma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(KT_SMEM_BYTES)));
    c->func_attr_mask |= attr_bit;
  }
  const bool vec_a = (K % 2 == 0) && (reinterpret_cast<uintptr_t>(A) % 8 == 0) && !getenv("VT_TMP_NOVEC");
  if (vec_a)
    sgemm_skinny_tma_kernel<true><<<ctas, KT_THREADS, KT_SMEM_BYTES, s>>>(tmB, A, C, partials, tickets, int(M), int(N),
                                                                         int(K), sc, c->status);
  else
    sgemm_skinny_tma_kernel<false><<<ctas, KT_THREADS, KT_SMEM_BYTES, s>>>(tmB, A, C, partials, tickets, int(M), int(N),
                                                                          int(K), sc, c->status);
  count_launch();
  VT_CUDA(cudaGetLastError());
  return VT_OK;
}

}  // namespace vt
