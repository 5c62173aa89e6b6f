// fp32 GEMM with few rows of A (a panel of up to 128) on the 5th-generation tensor cores: one stream of B.
//
// The product is computed transposed, C^T (n x m) = B^T (n x k) * A^T (k x m), so that the streamed
// matrix is the tensor core's 128-row operand:
//   A operand  a 32-row chunk of a 128-column slab of B exactly as it lies in memory (n contiguous:
//              an MN-major TF32 operand).  For 32-bit MN-major operands tcgen05 wants the
//              "128-byte swizzle with 32-byte atoms" layout: TMA boxes of 32 floats x 32 rows
//              written with that swizzle, descriptors with leading offset = one box (4 KiB) and
//              stride offset = four rows (512 B); a K step of 8 rows moves 1 KiB.
//   B operand  the matching MT x 32 block of A (k contiguous: K-major, plain 128-byte swizzle), MT
//              the panel height (16, 32, 64 or 128); rows past M are zero-filled by TMA.
//   D          128 lanes (n) x MT (or 2 x MT) columns of fp32 in tensor memory.
// fp32 accuracy comes from the 3xTF32 split, done without a pass over global memory.  The tensor
// core reads only the top 19 bits of each 32-bit operand, so the data as loaded *is* the hi part
// (cut, not rounded).  The lo parts, lo = x - hi (exact; its own cut-off point pre-rounded), are
// computed by warps of the CTA:
//   B lo  goes straight into tensor memory (tcgen05.st, 32 columns per chunk) and is used from
//         there as the A operand of its MMA, so B crosses shared memory once;
//   A lo  is written under A in shared memory, which makes [A; A lo] one operand of 2 x MT rows.
// Per K step of 8, stacked form:  B (smem) x [A; A lo] -> columns 0..MT-1 (hi*hi) and MT..2MT-1 (hi*lo);
//                                 B lo (tmem) x A      -> added into columns 0..MT-1 (lo*hi).
// (The unstacked form, B x A, B x A lo and B lo x A into one accumulator of MT columns, is kept as an
// option of the shape.)  Accumulators are folded into fp32 registers every few chunks (the tensor
// core's own accumulation truncates).
//
// The tall form (few columns of B against a large A) is the same pipeline with the roles exchanged; see
// KuShape below.
//
// One CTA per SM.  Warp 0 is the TMA producer (a ring of stages of B, A and room for A lo).  Small MMAs
// cost their issuing thread, and the warps that feed them, more time than the loads take, so
// the chunks of the ring are dealt to KU_PIPES independent pipes (chunk at ring position p goes to
// pipe p mod KU_PIPES).  A pipe is one MMA-issuing warp plus one or more sets of four splitting warps
// (one warp per TMEM lane quarter) with its own accumulators and B lo buffers; at the end of a piece of
// work the pipes' sums are added in pipe order through shared memory.  Work split and K-split
// reduction: see skinny_sched.cuh.  Every wait is bounded.
#include "ptx_sm100.cuh"
#include "runtime.h"
#include "skinny_sched.cuh"

namespace vt {
namespace {

constexpr int KU_CTAS_PER_SM = 1;
constexpr int KU_MAX_STAGES = 10;
constexpr int KU_MAX_PIPES = 2;
constexpr int KU_B_BYTES = SKINNY_KC * SKINNY_COLS * 4;   // 16 KiB: four boxes of 32 floats x 32 rows
constexpr int KU_BOX_BYTES = 32 * 32 * 4;
constexpr int KU_SMEM_LIMIT = 227 * 1024;

// One shape of the kernel:
//   MT       rows of A (the panel height, a multiple of 16 up to 128);
//   PIPES    independent pipes (MMA issuer, accumulators, B lo buffers, splitting warps);
//   SETS     sets of four splitting warps per pipe.  The pipe's chunks go to its sets in turn (the time a
//            set takes over a chunk is a chain of latencies, so sets overlap them), and every set drains
//            its own MT / SETS columns of each accumulator, so the running sums spread over the sets' registers;
//   STACKED  [A; A lo] as one operand of 2 * MT rows (two MMAs per K step, accumulators of 2 * MT columns:
//            [hi*hi | hi*lo]) or A and A lo as two operands into one accumulator of MT columns (three MMAs).
//   ACC_BUFS accumulators per pipe: two (one drained while the other fills) or one (the pipe's MMAs wait
//            while it is drained);
//   WINDOW   chunks a pipe accumulates in tensor memory between folds into registers.
// Tensor memory per pipe: the accumulators, then the B lo buffers of 32 columns each.
//   TALL     the mirror image, for C (M x N) = A (M x K) * B (K x N) with few columns (N <= MT) and A the
//            traffic: the streamed matrix is A, whose 128-row slabs are the tensor core's 128-row operand in the
//            ordinary K-major layout (so the product is not transposed and a TMEM lane is a row of C); the
//            small operand is [B | B lo], N-major as B lies in memory (MN-major TF32, the 32-byte-atom swizzle),
//            prepared once per call in a scratch array of K x 2 MT floats; the splitting warps write A lo to
//            tensor memory and have nothing to write to shared memory.
template <int MT, int PIPES, int SETS, bool STACKED, int ACC_BUFS, int WINDOW, bool TALL = false>
struct KuShape {
  static constexpr bool kTall = TALL;
  static constexpr int kRows = MT;
  static constexpr int kPipes = PIPES;
  static constexpr int kSets = SETS;
  static constexpr bool kStacked = STACKED;
  static constexpr int kAccBufs = ACC_BUFS;
  static constexpr int kWindow = WINDOW;
  static constexpr int kLoBufs = SETS < 2 ? 2 : SETS;
  static constexpr int kSetRows = MT / SETS;                        // accumulator columns one set drains
  static constexpr int kThreads = 32 * (1 + PIPES + 4 * PIPES * SETS);
  static constexpr int kABytes = MT * SKINNY_KC * 4;                // 2 KiB per 16 rows
  static constexpr int kStageBytes = KU_B_BYTES + 2 * kABytes;      // B, A, A lo
  static constexpr int kAccCols = STACKED ? 2 * MT : MT;
  static constexpr int kLoCol = kAccBufs * kAccCols;                // first B lo buffer; the others 32 columns on each
  static constexpr int kPipeCols = kLoCol + 32 * kLoBufs;
  static constexpr int kTmemCols = PIPES * kPipeCols <= 128 ? 128 : PIPES * kPipeCols <= 256 ? 256 : 512;
  static constexpr int kExchBytes = (PIPES - 1) * MT * SKINNY_COLS * 4;
  static constexpr int kFit = (KU_SMEM_LIMIT - 1024 - 512 - kExchBytes) / kStageBytes;
  static constexpr int kStages = kFit < KU_MAX_STAGES ? kFit : KU_MAX_STAGES;
  static constexpr size_t kSmemBytes = 1024 + size_t(kStages) * kStageBytes + kExchBytes + 512;
  // chunks' worth of time between two pieces of work (measured for the 16-row shape; the drain and
  // the result tile grow with the panel)
  static constexpr int kPieceOverhead = MT <= 16 ? 10 : MT <= 32 ? 10 : MT <= 64 ? 8 : 8;
  static_assert(MT % 16 == 0 && MT >= 16 && MT <= 128, "panel height");
  static_assert(PIPES >= 1 && PIPES <= KU_MAX_PIPES && SETS >= 1 && SETS <= 4, "pipes and sets");
  static_assert((ACC_BUFS == 1 || ACC_BUFS == 2) && WINDOW >= 1, "accumulators");
  static_assert(MT % SETS == 0 && kSetRows % 16 == 0, "a set drains whole groups of 16 columns");
  static_assert(kThreads <= 1024, "threads per CTA");
  static_assert(PIPES * kPipeCols <= 512, "tensor memory has 512 columns");
  static_assert(kStages >= 3, "the ring needs a few stages");
};

struct UmmaSkinnyPipe {
  uint64_t raw_full[KU_MAX_STAGES];    // TMA bytes have landed
  uint64_t split_done[KU_MAX_STAGES];  // the chunk's pipe has written the lo parts
  uint64_t empty[KU_MAX_STAGES];       // the MMAs that read the stage have retired
  uint64_t lo_free[KU_MAX_PIPES][4];   // the MMAs that read a B lo buffer in tensor memory have retired
  uint64_t acc_full[KU_MAX_PIPES][2];
  uint64_t acc_empty[KU_MAX_PIPES][2];
  uint32_t tmem_base;
  int abort_word;
  int last_flag;
};
static_assert(sizeof(UmmaSkinnyPipe) <= 512, "pipeline state has 512 bytes of shared memory");

// lo part of x as the tensor core should see it: x minus its top 19 bits, then half of the cut-off
// unit added to the bit pattern so that the core's own cut rounds to nearest.
__device__ __forceinline__ uint32_t lo_part(uint32_t bits) {
  const float hi = __uint_as_float(bits & 0xffffe000u);
  return __float_as_uint(__uint_as_float(bits) - hi) + 0x1000u;
}

template <class Shape>
__global__ void __launch_bounds__(Shape::kThreads, KU_CTAS_PER_SM)
sgemm_skinny_umma_kernel(const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmA,
                         float* __restrict__ C, float* __restrict__ partials, int* __restrict__ tickets, int M, int N,
                         int ldc, SkinnySched sc, int* __restrict__ status) {
  // Names follow the wide form (B streamed, A the small operand).  In the tall form `tmB` is the map of the
  // streamed matrix (A: boxes of 32 floats of K x 128 rows) and `tmA` that of the small one ([B | B lo]: boxes
  // of 32 columns x 32 rows of K); M and N are the rows and columns of C in both.  `ldc` is the row pitch of C
  // (tall form only: a launch may compute a panel of columns of a wider C; the partial tiles have pitch N).
  constexpr bool TALL = Shape::kTall;
  constexpr int MT = Shape::kRows;
  constexpr int KU_PIPES = Shape::kPipes;
  constexpr int KU_ACC_BUFS = Shape::kAccBufs;
  constexpr int KU_SETS = Shape::kSets;
  constexpr int KU_WINDOW = Shape::kWindow;
  constexpr int KU_LO_BUFS = Shape::kLoBufs;
  constexpr int MS = Shape::kSetRows;
  constexpr bool KU_STACKED = Shape::kStacked;
  constexpr int KU_STAGES = Shape::kStages;
  constexpr int KU_A_BYTES = Shape::kABytes;
  constexpr int KU_STAGE_BYTES = Shape::kStageBytes;
  constexpr int KU_PIPE_COLS = Shape::kPipeCols;
  constexpr int KU_ACC_COLS = Shape::kAccCols;
  constexpr int KU_LO_COL = Shape::kLoCol;
  constexpr int KU_TMEM_COLS = Shape::kTmemCols;
  constexpr int KU_EXCH_BYTES = Shape::kExchBytes;
  extern __shared__ uint8_t ku_smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ku_smem_raw) + 1023) & ~uintptr_t(1023));
  float* exch = reinterpret_cast<float*>(tiles + size_t(KU_STAGES) * KU_STAGE_BYTES);
  UmmaSkinnyPipe* ps = reinterpret_cast<UmmaSkinnyPipe*>(tiles + size_t(KU_STAGES) * KU_STAGE_BYTES + KU_EXCH_BYTES);
  volatile int* abort_word = &ps->abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = int(blockIdx.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < KU_STAGES; ++s) {
      mbar_init(&ps->raw_full[s], 1);
      mbar_init(&ps->split_done[s], 4);
      mbar_init(&ps->empty[s], 1);
    }
    for (int p = 0; p < KU_PIPES; ++p) {
      for (int b = 0; b < KU_LO_BUFS; ++b) mbar_init(&ps->lo_free[p][b], 1);
      for (int b = 0; b < KU_ACC_BUFS; ++b) {
        mbar_init(&ps->acc_full[p][b], 1);
        mbar_init(&ps->acc_empty[p][b], 4 * KU_SETS);
      }
    }
    ps->abort_word = 0;
    ps->last_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<1>(&ps->tmem_base, KU_TMEM_COLS);
    tmem_relinquish<1>();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmA);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ps->tmem_base;
  // Everything above may run while the kernel before this one on the stream is still finishing; nothing below
  // (operands, partial tiles, tickets, C, the status word) is touched before it has completed.
  grid_dependency_wait();
  grid_launch_dependents();

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t filled = 0, fill_parity = 0;
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      SkinnySegment seg;
      for (int idx = 0; ok && sched_segment(sc, cta, idx, seg); ++idx) {
        const int n0 = seg.slab * SKINNY_COLS;     // first column of B (wide) or first row of A (tall) of the slab
        for (int ch = seg.chunk_beg; ch < seg.chunk_end; ++ch) {
          if (!mbar_wait(&ps->empty[stage], phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_PRODUCER)) {
            ok = false;
            break;
          }
          uint64_t* full = &ps->raw_full[stage];
          uint8_t* dst = tiles + size_t(stage) * KU_STAGE_BYTES;
          if (TALL) {
            mbar_arrive_expect_tx(full, KU_B_BYTES + 2 * KU_A_BYTES);
            tma_load_2d(dst, &tmB, full, ch * SKINNY_KC, n0);
#pragma unroll
            for (int b = 0; b < 2 * MT / 32; ++b)
              tma_load_2d(dst + KU_B_BYTES + b * KU_BOX_BYTES, &tmA, full, 32 * b, ch * SKINNY_KC);
          } else {
            mbar_arrive_expect_tx(full, KU_B_BYTES + KU_A_BYTES);
#pragma unroll
            for (int b = 0; b < 4; ++b) tma_load_2d(dst + b * KU_BOX_BYTES, &tmB, full, n0 + 32 * b, ch * SKINNY_KC);
            tma_load_2d(dst + KU_B_BYTES, &tmA, full, ch * SKINNY_KC, 0);
          }
          filled |= 1u << stage;
          fill_parity = (fill_parity & ~(1u << stage)) | (phase << stage);
          if (++stage == KU_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (ok) {
        // Tail: every stage released => every MMA that reads shared memory has retired and every
        // commit arrival has landed before the CTA gives its shared memory back.
        for (int s = 0; s < KU_STAGES; ++s) {
          if (!mbar_wait(&ps->empty[stage], phase ^ 1, abort_word, KSTAT_WAIT_EXPIRED_PRODUCER)) break;
          if (++stage == KU_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (*abort_word != 0) {
        // Aborting: wait (bounded) for the copies already issued before shared memory goes back.
        for (int s = 0; s < KU_STAGES; ++s)
          if (filled & (1u << s)) mbar_wait_drain(&ps->raw_full[s], (fill_parity >> s) & 1u);
      }
    }
    __syncwarp();
  } else if (warp <= KU_PIPES) {
    // ------------------------------ MMA issuer of pipe (warp - 1) ------------------------------
    if (lane == 0) {
      const int pipe = warp - 1;
      // wide: 128-row operand MN-major (B as stored), small operand K-major; tall: 128-row operand K-major
      // (A as stored), small operand MN-major ([B | B lo] as stored)
      constexpr uint32_t idesc_pair =
          umma_instr_desc(UMMA_D_F32, UMMA_AB_TF32, !TALL, TALL, 128, KU_STACKED ? 2 * MT : MT);
      constexpr uint32_t idesc_lo = umma_instr_desc(UMMA_D_F32, UMMA_AB_TF32, false, TALL, 128, MT);
      // Descriptors are kept as a constant high word and a low word that only ever has a constant
      // added to it, and the ring position is counted, not divided.
      constexpr uint32_t kMn32Hi = (512u >> 4) | (1u << 14) | (1u << 29);    // stride offset, version, swizzle mode 1
      constexpr uint32_t kSw128Hi = (1024u >> 4) | (1u << 14) | (2u << 29);  // stride offset, version, swizzle mode 2
      const uint32_t tiles_lo = (smem_u32(tiles) & 0x3FFFFu) >> 4;
      auto make_desc = [](uint32_t lo, uint32_t hi) {
        uint64_t d;
        asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
        return d;
      };
      const uint32_t pipe_tmem = tmem_base + uint32_t(pipe * KU_PIPE_COLS);
      uint32_t stage = 0, phase = 0, turn = 0;   // ring position of the next chunk; turn = position mod KU_PIPES
      uint32_t mine = 0;                         // chunks this pipe has taken: B lo buffer = mine mod KU_LO_BUFS
      int win = 0;
      bool ok = true;
      SkinnySegment seg;
      for (int idx = 0; ok && sched_segment(sc, cta, idx, seg); ++idx) {
        const int nchunks = seg.chunk_end - seg.chunk_beg;
        int in_window = 0;
        for (int i = 0; i < nchunks; ++i) {
          if (int(turn) == pipe) {
            const int buf = win % KU_ACC_BUFS;
            const uint32_t lo_buf = mine % KU_LO_BUFS;
            const bool opens = in_window == 0;
            if (opens && !mbar_wait(&ps->acc_empty[pipe][buf], (uint32_t(win / KU_ACC_BUFS) & 1u) ^ 1u, abort_word,
                                    KSTAT_WAIT_EXPIRED_MMA)) {
              ok = false;
              break;
            }
            if (!mbar_wait(&ps->split_done[stage], phase, abort_word, KSTAT_WAIT_EXPIRED_MMA)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t b_lo32 = (tiles_lo + stage * (KU_STAGE_BYTES >> 4)) | ((4096u >> 4) << 16);            // B as loaded
            const uint32_t a_lo32 = (tiles_lo + stage * (KU_STAGE_BYTES >> 4) + (KU_B_BYTES >> 4)) | (1u << 16);  // [A; A lo]
            const uint32_t d_tmem = pipe_tmem + uint32_t(buf * KU_ACC_COLS);
            const uint32_t lo_tmem = pipe_tmem + uint32_t(KU_LO_COL) + lo_buf * 32u;
#pragma unroll
            for (int ks = 0; ks < SKINNY_KC / 8; ++ks) {
              if (TALL) {
                static_assert(!TALL || KU_STACKED, "the tall form is stacked");
                // streamed A: K-major, 32 bytes per K step; [B | B lo]: N-major boxes, 1 KiB (8 rows) per K step
                const uint64_t big = make_desc(((tiles_lo + stage * (KU_STAGE_BYTES >> 4)) | (1u << 16)) + ks * (32u >> 4), kSw128Hi);
                const uint64_t small = make_desc(
                    ((tiles_lo + stage * (KU_STAGE_BYTES >> 4) + (KU_B_BYTES >> 4)) | ((4096u >> 4) << 16)) + ks * (1024u >> 4), kMn32Hi);
                umma_tf32<1>(d_tmem, big, small, idesc_pair, (ks == 0 && opens) ? 0u : 1u);
                umma_tf32_a_tmem(d_tmem, lo_tmem + uint32_t(ks * 8), small, idesc_lo, 1u);
                continue;
              }
              const uint64_t a_desc = make_desc(a_lo32 + ks * (32u >> 4), kSw128Hi);
              const uint64_t b_desc = make_desc(b_lo32 + ks * (1024u >> 4), kMn32Hi);
              umma_tf32<1>(d_tmem, b_desc, a_desc, idesc_pair, (ks == 0 && opens) ? 0u : 1u);
              if (!KU_STACKED) {
                const uint64_t a_lo_desc = make_desc(a_lo32 + (uint32_t(KU_A_BYTES) >> 4) + ks * (32u >> 4), kSw128Hi);
                umma_tf32<1>(d_tmem, b_desc, a_lo_desc, idesc_pair, 1u);
              }
              umma_tf32_a_tmem(d_tmem, lo_tmem + uint32_t(ks * 8), a_desc, idesc_lo, 1u);
            }
            umma_commit(&ps->empty[stage]);
            umma_commit(&ps->lo_free[pipe][lo_buf]);
            // The window closes when it is full or with this pipe's last chunk of the piece.
            if (++in_window == KU_WINDOW || i + KU_PIPES >= nchunks) {
              umma_commit(&ps->acc_full[pipe][buf]);
              ++win;
              in_window = 0;
            }
            ++mine;
          }
          if (++turn == KU_PIPES) turn = 0;
          if (++stage == KU_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else {
    // ------------- splitting warps of a pipe: lo parts, accumulator drain, result -------------
    const int pipe = (warp - 1 - KU_PIPES) / (4 * KU_SETS);
    const int set = ((warp - 1 - KU_PIPES) >> 2) % KU_SETS;
    const int quarter = warp & 3;                                 // the TMEM lanes (and the TMA box) of this warp
    const int t = ((warp - 1 - KU_PIPES) & 3) * 32 + lane;        // 0..127 within the set
    const uint32_t lane_base = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(pipe * KU_PIPE_COLS);
    uint32_t stage = 0, phase = 0, turn = 0, mine = 0;
    int win = 0;
    bool ok = true;
    SkinnySegment seg;
    for (int idx = 0; sched_segment(sc, cta, idx, seg); ++idx) {
      const int nchunks = seg.chunk_end - seg.chunk_beg;
      float master[MS];            // rows set * MS .. + MS of the panel, at this thread's column of the slab
#pragma unroll
      for (int m = 0; m < MS; ++m) master[m] = 0.f;
      // Adds this set's columns of the pipe's oldest undrained accumulator into master.
      auto drain = [&]() -> bool {
        const int buf = win % KU_ACC_BUFS;
        // Every lane polls; the vote brings the warp back together before the warp-wide tcgen05 operations.
        if (!__all_sync(0xffffffffu, mbar_wait(&ps->acc_full[pipe][buf], uint32_t(win / KU_ACC_BUFS) & 1u, abort_word,
                                               KSTAT_WAIT_EXPIRED_EPILOGUE)))
          return false;
        tc_fence_after_sync();
#pragma unroll
        for (int g = 0; g < MS / 16; ++g) {
          const uint32_t col = lane_base + uint32_t(buf * KU_ACC_COLS + set * MS + g * 16);
          uint32_t r0[16];
          tmem_ld_32x32b_x16(col, r0);
          if (KU_STACKED) {
            uint32_t r1[16];
            tmem_ld_32x32b_x16(col + uint32_t(MT), r1);
            tmem_ld_wait();
#pragma unroll
            for (int m = 0; m < 16; ++m) master[g * 16 + m] += __uint_as_float(r0[m]) + __uint_as_float(r1[m]);
          } else {
            tmem_ld_wait();
#pragma unroll
            for (int m = 0; m < 16; ++m) master[g * 16 + m] += __uint_as_float(r0[m]);
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ps->acc_empty[pipe][buf]);
        ++win;
        return true;
      };
      int seen = 0, drained = 0;   // chunks of this pipe so far in the piece; accumulators this set has drained
      for (int i = 0; i < nchunks && ok; ++i) {
        if (int(turn) == pipe && int(mine % KU_SETS) != set) {
          ++seen;
          ++mine;
        } else if (int(turn) == pipe) {
          ok = __all_sync(0xffffffffu, mbar_wait(&ps->raw_full[stage], phase, abort_word, KSTAT_WAIT_EXPIRED_EPILOGUE));
          if (!ok) break;
          const uint8_t* stage_ptr = tiles + size_t(stage) * KU_STAGE_BYTES;
          // This thread's column of the slab, all 32 rows of the chunk.  Box `quarter`: rows of
          // 128 bytes, 32-byte units XOR-swizzled with (row % 4).
          const float* box = reinterpret_cast<const float*>(stage_ptr + quarter * KU_BOX_BYTES);
          uint32_t lo_a[16], lo_b[16];
          if (TALL) {
            // This thread's row of the slab: 128 bytes, 16-byte units XOR-swizzled with (row % 8).
            const int row = quarter * 32 + lane;
            const uint32_t row_addr = smem_u32(stage_ptr) + uint32_t(row) * 128u;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              uint32_t x0, x1, x2, x3;
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3)
                           : "r"(row_addr + (uint32_t(u ^ (row & 7)) << 4)));
              uint32_t* out = u < 4 ? &lo_a[4 * u] : &lo_b[4 * (u - 4)];
              out[0] = lo_part(x0);
              out[1] = lo_part(x1);
              out[2] = lo_part(x2);
              out[3] = lo_part(x3);
            }
          } else {
#pragma unroll
          for (int k = 0; k < 16; ++k)
            lo_a[k] = lo_part(__float_as_uint(box[k * 32 + (((lane >> 3) ^ (k & 3)) << 3) + (lane & 7)]));
#pragma unroll
          for (int k = 16; k < 32; ++k)
            lo_b[k - 16] = lo_part(__float_as_uint(box[k * 32 + (((lane >> 3) ^ (k & 3)) << 3) + (lane & 7)]));
          }
#pragma unroll
          for (int v = 0; v < (TALL ? 0 : MT / 16); ++v) {
            // A lo under A, position for position (both blocks carry the same swizzle)
            const uint32_t a_addr = smem_u32(stage_ptr + KU_B_BYTES) + uint32_t(v * 128 + t) * 16u;
            uint32_t x0, x1, x2, x3;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3) : "r"(a_addr));
            st_shared_v4(a_addr + KU_A_BYTES, lo_part(x0), lo_part(x1), lo_part(x2), lo_part(x3));
          }
          // The MMAs that read this B lo buffer KU_LO_BUFS of this pipe's chunks ago must have retired.
          const uint32_t lo_buf = mine % KU_LO_BUFS;
          ok = __all_sync(0xffffffffu, mbar_wait(&ps->lo_free[pipe][lo_buf], (uint32_t(mine / KU_LO_BUFS) & 1u) ^ 1u,
                                                 abort_word, KSTAT_WAIT_EXPIRED_EPILOGUE));
          if (!ok) break;
          tc_fence_after_sync();
          tmem_st_32x32b_x16(lane_base + uint32_t(KU_LO_COL) + lo_buf * 32u, lo_a);
          tmem_st_32x32b_x16(lane_base + uint32_t(KU_LO_COL) + lo_buf * 32u + 16u, lo_b);
          tmem_st_wait();
          fence_proxy_async_smem();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ps->split_done[stage]);
          // Accumulators that closed before this chunk have had this whole split to finish.
          while (ok && drained < seen / KU_WINDOW) {
            ok = drain();
            ++drained;
          }
          ++seen;
          ++mine;
        }
        if (++turn == KU_PIPES) turn = 0;
        if (++stage == KU_STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
      const int windows = (seen + KU_WINDOW - 1) / KU_WINDOW;
      while (ok && drained < windows) {
        ok = drain();
        ++drained;
      }

      // Pipes above 0 hand their sums to pipe 0, which adds them in pipe order.  Whether the CTA is
      // giving up is read between the two barriers, where no thread can still be in a wait, so all
      // splitting threads take the same way out.
      if (KU_PIPES > 1 && pipe > 0) {
#pragma unroll
        for (int m = 0; m < MS; ++m) exch[((pipe - 1) * MT + set * MS + m) * SKINNY_COLS + t] = master[m];
      }
      asm volatile("bar.sync 2, %0;" ::"n"(128 * KU_PIPES * KU_SETS) : "memory");
      const bool giving_up = *abort_word != 0;
      if (pipe == 0) {
#pragma unroll
        for (int q = 1; q < KU_PIPES; ++q)
#pragma unroll
          for (int m = 0; m < MS; ++m) master[m] += exch[((q - 1) * MT + set * MS + m) * SKINNY_COLS + t];
      }
      asm volatile("bar.sync 2, %0;" ::"n"(128 * KU_PIPES * KU_SETS) : "memory");   // exch may be rewritten
      if (giving_up) break;
      if (pipe == 0) {
        // The tile of this piece goes to C (the slab has one piece) or to its slot among the slab's partial tiles.
        float* dst = seg.parts == 1 ? C : partials + size_t(seg.part) * size_t(M) * size_t(N);
        const int col = seg.slab * SKINNY_COLS + quarter * 32 + lane;
        if (TALL) {
          // `col` is this thread's row of C; its MS sums are consecutive columns of that row
          if (col < M) {
            const size_t pitch = seg.parts == 1 ? size_t(ldc) : size_t(N);
#pragma unroll
            for (int m = 0; m < MS; ++m)
              if (set * MS + m < N) dst[size_t(col) * pitch + set * MS + m] = master[m];
          }
          if (seg.parts > 1) {
            const int rows = M - seg.slab * SKINNY_COLS < SKINNY_COLS ? M - seg.slab * SKINNY_COLS : SKINNY_COLS;
            skinny_finish_block<128 * KU_SETS>(seg, set * 128 + t, 1, &ps->last_flag, tickets, partials, C,
                                               size_t(M) * size_t(N), seg.slab * SKINNY_COLS, rows, N, ldc);
          }
        } else {
        if (col < N) {
#pragma unroll
          for (int m = 0; m < MS; ++m)
            if (set * MS + m < M) dst[size_t(set * MS + m) * N + col] = master[m];
        }
        if (seg.parts > 1)
          skinny_finish_piece<128 * KU_SETS, MT>(seg, set * 128 + t, 1, &ps->last_flag, tickets, partials, C, M, N);
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc<1>(tmem_base, KU_TMEM_COLS);
  if (threadIdx.x == 0 && ps->abort_word != 0) atomicCAS(status, 0, ps->abort_word);
}

// The shapes the library builds, by panel height.  Small MMAs are bound by their issuing thread, hence
// two pipes while tensor memory has room for them (2 x (2 x 2*MT + 64) columns); the 128-row panel
// fills one accumulator of 256 columns per pipe and drains it in place.
// Measured at 8192^2 / 4096^2 / 1024^2 elements of B, in us.  64 rows: one pipe of two sets 83 / 31 / 15, two pipes
// of one accumulator each 74 / 34 / 19.  128 rows: 107-109 / 42-45 in every form tried: stacked with one
// accumulator (this one, the most accurate), unstacked with two, A lo loaded from a pass over A instead of
// computed here, B itself copied to tensor memory so that no MMA reads it from shared memory, waits that keep
// draining finished accumulators, and (timing only) a six-stage ring.  What bounds it is the one thread that
// issues the MMAs: about 700 cycles per chunk for eight MMAs and two commits, plus its waits for the lo parts
// and for the drained accumulator, against 800 cycles of tensor-core work.  The same pipeline on CTA pairs
// (cta_group::2: one MMA of 256 rows for two neighbouring slabs, the N-side split between the CTAs made to
// coincide with the A / A lo split) was built and was bit-for-bit as accurate, but slower: 143 us at 128 rows,
// 130 us at 64; its issuing thread spent 630 cycles per chunk pair issuing and 1000-1100 waiting for lo parts
// and drained accumulators that cross the cluster.
using KuShape16 = KuShape<16, 2, 1, true, 2, 4>;
using KuShape32 = KuShape<32, 2, 1, true, 2, 4>;
using KuShape64 = KuShape<64, 1, 2, true, 2, 4>;
using KuShape64Large = KuShape<64, 2, 1, true, 1, 4>;     // from 32 Mi elements of B
using KuShape128 = KuShape<128, 1, 2, true, 1, 4>;

template <class Shape>
int launch_shape(DeviceCtx* c, uint32_t attr_bit, const float* A, const float* B, float* C, float* partials, int* tickets,
                 int64_t M, int64_t N, int64_t K, cudaStream_t s) {
  int ctas;
  const SkinnySched sc = make_skinny_sched(N, K, c->sm_count, KU_CTAS_PER_SM, Shape::kPieceOverhead, &ctas);
  if (skinny_max_parts(sc) > 1 && (!partials || !tickets)) return fail(VT_ERR_INVALID, "skinny K split needs scratch memory");
  if (sc.slabs > kTicketCount)
    return fail(VT_ERR_UNSUPPORTED, "N = %lld has more slabs than the library keeps tickets for", (long long)N);
  CUtensorMap tmB, tmA;
  int rc = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, B, uint64_t(N), uint64_t(K), uint64_t(N) * 4, 32, 32,
                          CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  if (rc) return rc;
  rc = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, A, uint64_t(K), uint64_t(M), uint64_t(K) * 4, 32,
                      Shape::kRows);
  if (rc) return rc;
  if (!(c->func_attr_mask & attr_bit)) {
    VT_CUDA(cudaFuncSetAttribute(sgemm_skinny_umma_kernel<Shape>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(Shape::kSmemBytes)));
    c->func_attr_mask |= attr_bit;
  }
  VT_CUDA(launch_overlapped(sgemm_skinny_umma_kernel<Shape>, unsigned(ctas), unsigned(Shape::kThreads),
                            size_t(Shape::kSmemBytes), s, tmB, tmA, C, partials, tickets, int(M), int(N), int(N), sc,
                            c->status));
  count_launch();
  VT_CUDA(cudaGetLastError());
  return VT_OK;
}

// Tall form: up to 16, 32 or 64 columns of C.
using KuTall16 = KuShape<16, 2, 1, true, 2, 4, true>;
using KuTall32 = KuShape<32, 2, 1, true, 2, 4, true>;
using KuTall64 = KuShape<64, 1, 2, true, 2, 4, true>;
using KuTall64Large = KuShape<64, 2, 1, true, 1, 4, true>;   // from 32 Mi elements of A
using KuTall128 = KuShape<128, 1, 2, true, 1, 4, true>;

// [B | B lo] for the tall form: row k holds B[k][0..N) padded with zeros to `nt` columns, then their lo parts.
// (B has row pitch `ldb`; the N columns are a panel of it.)
__global__ void __launch_bounds__(256) tall_b_and_lo_kernel(const float* __restrict__ B, float* __restrict__ out, int64_t K,
                                                            int N, int nt, int64_t ldb) {
  // Launched for overlap with the kernel before it: `out` is scratch that the streaming kernel of the previous
  // panel or call may still be reading, so nothing is touched before that kernel has completed.
  grid_dependency_wait();
  grid_launch_dependents();
  const int64_t total = K * 2 * nt;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t k = i / (2 * nt);
    const int j = int(i - k * 2 * nt);
    const int col = j < nt ? j : j - nt;
    float v = 0.f;
    if (col < N) {
      v = B[k * ldb + col];
      if (j >= nt) v = __uint_as_float(lo_part(__float_as_uint(v)));
    }
    out[i] = v;
  }
}

template <class Shape>
int launch_tall_shape(DeviceCtx* c, uint32_t attr_bit, const float* A, const float* B, float* C, float* partials,
                      int* tickets, float* b_and_lo, int64_t M, int64_t N, int64_t K, int64_t ldb, int64_t ldc,
                      cudaStream_t s) {
  constexpr int NT = Shape::kRows;
  int ctas;
  const SkinnySched sc = make_skinny_sched(M, K, c->sm_count, KU_CTAS_PER_SM, Shape::kPieceOverhead, &ctas);
  if (skinny_max_parts(sc) > 1 && (!partials || !tickets)) return fail(VT_ERR_INVALID, "tall K split needs scratch memory");
  if (sc.slabs > kTicketCount)
    return fail(VT_ERR_UNSUPPORTED, "M = %lld has more slabs than the library keeps tickets for", (long long)M);
  const int64_t total = K * 2 * NT;
  const int blocks = int(total / 256 + 1 < int64_t(c->sm_count) * 8 ? total / 256 + 1 : int64_t(c->sm_count) * 8);
  VT_CUDA(launch_overlapped(tall_b_and_lo_kernel, unsigned(blocks), 256u, size_t(0), s, B, b_and_lo, K, int(N), int(NT),
                            ldb));
  count_launch();
  CUtensorMap tmBig, tmSmall;
  int rc = encode_tmap_2d(&tmBig, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, A, uint64_t(K), uint64_t(M), uint64_t(K) * 4, 32, 128);
  if (rc) return rc;
  rc = encode_tmap_2d(&tmSmall, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, b_and_lo, uint64_t(2 * NT), uint64_t(K),
                      uint64_t(2 * NT) * 4, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  if (rc) return rc;
  if (!(c->func_attr_mask & attr_bit)) {
    VT_CUDA(cudaFuncSetAttribute(sgemm_skinny_umma_kernel<Shape>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(Shape::kSmemBytes)));
    c->func_attr_mask |= attr_bit;
  }
  VT_CUDA(launch_overlapped(sgemm_skinny_umma_kernel<Shape>, unsigned(ctas), unsigned(Shape::kThreads),
                            size_t(Shape::kSmemBytes), s, tmBig, tmSmall, C, partials, tickets, int(M), int(N), int(ldc),
                            sc, c->status));
  count_launch();
  VT_CUDA(cudaGetLastError());
  return VT_OK;
}

int piece_overhead_for(int64_t M) {
  return M <= 16 ? KuShape16::kPieceOverhead : M <= 32 ? KuShape32::kPieceOverhead
         : M <= 64 ? KuShape64::kPieceOverhead : KuShape128::kPieceOverhead;
}

}  // namespace

void sgemm_skinny_umma_plan(int64_t M, int64_t N, int64_t K, int sm_count, int* ctas, int* slabs, int* max_parts) {
  const SkinnySched sc = make_skinny_sched(N, K, sm_count, KU_CTAS_PER_SM, piece_overhead_for(M), ctas);
  *slabs = sc.slabs;
  *max_parts = skinny_max_parts(sc);
}

// Tall form: a panel of up to 128 columns of C (M x N, row pitch ldc) = A (M x K) * the same columns of B (row pitch
// ldb), A streamed once per panel.
int sgemm_tall_umma_panel(int64_t N) { return N <= 16 ? 16 : N <= 32 ? 32 : N <= 64 ? 64 : 128; }

void sgemm_tall_umma_plan(int64_t M, int64_t N, int64_t K, int sm_count, int* max_parts, size_t* b_and_lo_bytes) {
  int ctas;
  const int overhead = N <= 16 ? KuTall16::kPieceOverhead : N <= 32 ? KuTall32::kPieceOverhead
                       : N <= 64 ? KuTall64::kPieceOverhead : KuTall128::kPieceOverhead;
  const SkinnySched sc = make_skinny_sched(M, K, sm_count, KU_CTAS_PER_SM, overhead, &ctas);
  *max_parts = skinny_max_parts(sc);
  *b_and_lo_bytes = size_t(K) * 2 * size_t(sgemm_tall_umma_panel(N)) * 4;
}

bool sgemm_tall_umma_supported(const float* A, const float* B, const float* C, int64_t M, int64_t N, int64_t K) {
  (void)B;
  // one arrival counter per 128-row slab of A
  return N >= 4 && N % 4 == 0 && M >= 1 && M <= int64_t(kTicketCount) * SKINNY_COLS && K % 4 == 0 && K >= 4 &&
         K < (1LL << 31) && N < (1LL << 31) &&
         ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(C)) & 15) == 0;
}

int launch_sgemm_tall_umma(DeviceCtx* c, const float* A, const float* B, float* C, float* partials, int* tickets,
                           float* b_and_lo, int64_t M, int64_t N, int64_t K, int64_t ldb, int64_t ldc, cudaStream_t s) {
  if (!sgemm_tall_umma_supported(A, B, C, M, N, K) || N > SKINNY_UMMA_MAX_ROWS || ldc % 4 != 0)
    return fail(VT_ERR_UNSUPPORTED,
                "tall tensor-core kernel needs panels of N <= 128, N %% 4 == 0, K %% 4 == 0 and 16-byte aligned A and C");
  if (!b_and_lo) return fail(VT_ERR_INVALID, "tall kernel needs scratch memory for [B | B lo]");
  if (N <= 16) return launch_tall_shape<KuTall16>(c, 1u << 26, A, B, C, partials, tickets, b_and_lo, M, N, K, ldb, ldc, s);
  if (N <= 32) return launch_tall_shape<KuTall32>(c, 1u << 27, A, B, C, partials, tickets, b_and_lo, M, N, K, ldb, ldc, s);
  if (N > 64) return launch_tall_shape<KuTall128>(c, 1u << 30, A, B, C, partials, tickets, b_and_lo, M, N, K, ldb, ldc, s);
  if (double(M) * double(K) >= 3.2e7)
    return launch_tall_shape<KuTall64Large>(c, 1u << 29, A, B, C, partials, tickets, b_and_lo, M, N, K, ldb, ldc, s);
  return launch_tall_shape<KuTall64>(c, 1u << 28, A, B, C, partials, tickets, b_and_lo, M, N, K, ldb, ldc, s);
}

bool sgemm_skinny_umma_supported(const float* A, const float* B, const float* C, int64_t M, int64_t N, int64_t K) {
  // one arrival counter per 128-column slab of B
  return M >= 1 && M <= SKINNY_UMMA_MAX_ROWS && N % 4 == 0 && N >= 4 && N <= int64_t(kTicketCount) * SKINNY_COLS &&
         K % 4 == 0 && K >= 4 && K < (1LL << 31) &&
         ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) == 0;
}

int launch_sgemm_skinny_umma(DeviceCtx* c, const float* A, const float* B, float* C, float* partials, int* tickets,
                             int64_t M, int64_t N, int64_t K, cudaStream_t s) {
  if (!sgemm_skinny_umma_supported(A, B, C, M, N, K))
    return fail(VT_ERR_UNSUPPORTED,
                "row-panel tensor-core kernel needs M <= %d, N %% 4 == 0, K %% 4 == 0 and 16-byte aligned operands",
                SKINNY_UMMA_MAX_ROWS);
  if (M <= 16) return launch_shape<KuShape16>(c, 1u << 21, A, B, C, partials, tickets, M, N, K, s);
  if (M <= 32) return launch_shape<KuShape32>(c, 1u << 22, A, B, C, partials, tickets, M, N, K, s);
  if (M <= 64 && double(N) * double(K) >= 3.2e7)
    return launch_shape<KuShape64Large>(c, 1u << 25, A, B, C, partials, tickets, M, N, K, s);
  if (M <= 64) return launch_shape<KuShape64>(c, 1u << 23, A, B, C, partials, tickets, M, N, K, s);
  return launch_shape<KuShape128>(c, 1u << 24, A, B, C, partials, tickets, M, N, K, s);
}

}  // namespace vt
