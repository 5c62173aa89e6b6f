/* veritac_b200 — C ABI of the B200 (sm_100a) GEMM backend for VeriTac's CodeGen hot path.
 *
 * The reference (CuteCake/VeriTac) has no FFI: its two GEMM back ends are Python modules that
 * interpret or compile-and-run the computation on the CPU.  Each entry point below names the
 * reference interface whose execution it replaces.  Everything is plain pointers and sizes;
 * matrices are dense row-major with no padding (lda = K, ldb = N, ldc = N) and C is overwritten
 * (beta = 0), matching the reference, which poisons C and demands that every cell be written
 * (specializations/gemmini_gemm/backend.py:558-561, :756-760).
 *
 * Conventions
 *   - Every function returns VT_OK (0) or a negative VT_ERR_* code and never aborts the process;
 *     the text for the calling thread's last failure is vt_last_error().
 *   - `dev` is a CUDA device ordinal.  The library keeps one context per device (a stream, a status
 *     word, grow-only workspace) created on first use and freed by vt_shutdown().  A call that takes
 *     `dev` makes it the calling thread's current CUDA device and leaves it so, as cudaSetDevice(dev)
 *     would (a caller that allocates on "the current device" afterwards allocates there); the two
 *     calls that only answer a question or use a fixed array, vt_sgemm_auto_variant and
 *     vt_sgemm_skinny_static_scratch, put the previous device back.
 *   - `where`: VT_HOST  = A, B, C are host pointers; the call copies in, computes, copies out and
 *                         returns when C is complete (pinned memory from vt_host_alloc makes the
 *                         copies run at full PCIe rate).
 *              VT_DEVICE = A, B, C are device pointers on `dev`; the call only enqueues work on
 *                         `stream` (a cudaStream_t, or NULL for the library's own stream; the
 *                         legacy default stream is cudaStreamLegacy, (void*)1) and returns;
 *                         vt_sync() waits and reports kernel status.
 *              VT_HOST_AC_DEVICE_B (vt_i8gemm only) = one rank of a row-sharded job: A and C are this
 *                         rank's row blocks in host memory, B is the replicated operand, already in
 *                         this GPU's memory once the work queued on `stream` has run (the broadcast
 *                         that delivered it).  Copies A in, computes, copies C out and returns when C
 *                         is complete, like VT_HOST.
 *   - One host thread per device at a time; different devices may be driven concurrently.
 *   - All calls on one device must be ordered with one another on the GPU (the same stream, or streams joined
 *     by events): they share the device's status word, arrival counters and scratch memory (K-split partial
 *     tiles, lo parts), so two calls whose kernels could overlap race on them.
 *   - A VT_DEVICE call that needs more scratch memory than any call before it on that device grows the
 *     workspace, which synchronises the device and allocates; issue the largest shape once before
 *     latency-critical work or stream capture.
 */
#ifndef VERITAC_B200_H
#define VERITAC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  VT_OK = 0,
  VT_ERR_INVALID = -1,     /* bad argument: null pointer, shape outside the Gemmini plan domain, ... */
  VT_ERR_CUDA = -2,        /* a CUDA runtime/driver call failed; text in vt_last_error() */
  VT_ERR_DEVICE_WAIT = -3, /* a bounded device-side wait expired; the kernel returned early */
  VT_ERR_UNSUPPORTED = -4, /* variant not available for these arguments */
  VT_ERR_OVERFLOW = -5,    /* tile program could leave the int32 accumulator range */
  VT_ERR_PROGRAM = -6      /* malformed tile program */
};

enum { VT_HOST = 0, VT_DEVICE = 1, VT_HOST_AC_DEVICE_B = 2 };

/* Tile visiting order of the int8 GEMM = the loop order of the Gemmini schedule it stands for.
 * The order affects cache reuse only; results are identical for all of them. */
enum {
  VT_RASTER_BASELINE = 0, /* gen_baseline i,j,k   (backend.py:278-302): row-major output tiles      */
  VT_RASTER_REUSE_B = 1,  /* gen_reuse_b  j,k,i   (backend.py:305-333): column-major output tiles   */
  VT_RASTER_BATCHED = 2,  /* gen_batched_reuse_b  (lowering.py:18-40): batch_rows 16-row tiles of one
                             column block stay live together; columns swept per row batch         */
  VT_RASTER_AUTO = 3      /* grouped order tuned for L2 reuse on B200                               */
};

/* int8 kernel variants.  VT_I8_AUTO picks the fastest verified one (CTA_PAIR above 128 rows); the others
 * exist so that a design choice can be measured against its alternative:
 *   B_AS_STORED            one CTA per 128x256 tile
 *   CTA_PAIR               two CTAs per 256x256 tile (tcgen05 cta_group::2), every tile computed by one pair
 *   CTA_PAIR_WIDE          two CTAs per 256x512 tile: both halves share the pair's rows of A, which cuts the
 *                          operand traffic per product by a quarter; tensor memory is then full, so a tile's
 *                          epilogue does not overlap the next tile's MMAs.  For products of few tiles per pair
 *                          (row shards of a multi-GPU job).
 * All read B as stored and write C by TMA stores. */
enum {
  VT_I8_AUTO = 0,
  VT_I8_B_AS_STORED = 1,
  VT_I8_CTA_PAIR = 3,      /* 2 and 5 were forms that shared the last round of tiles along K: measured level, retired */
  VT_I8_CTA_PAIR_WIDE = 4
};

/* fp32 kernel variants.
 *   TILE128 / TILE64  register-tiled FFMA kernel (true fp32 arithmetic), 128x128 or 64x64 CTA tiles
 *   PIPE128 / PIPE64X128 / PIPE64
 *                     true fp32 FFMA as well, second design: 128x128, 64x128 or 64x64 CTA tiles fed by a
 *                     three-stage cp.async ring in the operands' own layout, 8x8 outputs per thread as packed pairs
 *                     (fma.rn.f32x2); with few tiles K is split over the CTAs of a thread-block cluster, which add
 *                     their partial tiles through each other's shared memory, in a fixed order: the mid-sized
 *                     products, where the first design leaves SMs idle (N % 4 == 0, K % 4 == 0, 16-byte aligned
 *                     operands)
 *   TILE32            32x32 CTA tiles, K brought in 256 at a time and split four ways inside the CTA (true fp32):
 *                     for products too small to fill the GPU with 64x64 tiles (N % 4 == 0, K % 4 == 0, aligned)
 *   SKINNY            M <= 16, N % 4 == 0: streams B once (HBM-bound), true fp32 FFMA arithmetic
 *   TF32X3            tensor cores, every operand split into TF32 hi + lo, three MMAs per product
 *                     (N % 4 == 0, K % 4 == 0, 16-byte aligned operands)
 *   SKINNY_TF32X3     M <= 16 on the tensor cores (3xTF32): one TMA-fed launch, tcgen05 with B used as it
 *                     lies in memory; when K % 4 != 0 or A is not 16-byte aligned, SKINNY_MMA_SYNC runs
 *   SKINNY_MMA_SYNC   the same stream of B with the products on mma.sync TF32 (any K, any alignment of A)
 *   TALL_TF32X3       the mirror image of PANEL_TF32X3 for few columns (N % 4 == 0, K % 4 == 0, 16-byte aligned A
 *                     and C): A is streamed once per panel of up to 128 columns, 128 rows at a time, against
 *                     [B | B lo] of the panel
 *   (3xTF32 forms and non-finite inputs: x * inf is formed as hi * inf + lo * inf, which is NaN where lo is zero
 *    or of the other sign; where an operand row or column holds an infinity, the TILE* and SKINNY variants give
 *    the IEEE result and the 3xTF32 forms may give NaN in its place.)
 *   PANEL_TF32X3      the SKINNY_TF32X3 kernel with taller panels of A (16, 32, 64 or 128 rows per launch, one
 *                     launch per 128 rows of A), for products with few rows where B is the traffic
 *                     (N % 4 == 0, K % 4 == 0, 16-byte aligned operands) */
enum {
  VT_SGEMM_AUTO = 0,
  VT_SGEMM_TILE128 = 1,
  VT_SGEMM_TILE64 = 2,
  VT_SGEMM_SKINNY = 3,
  VT_SGEMM_TF32X3 = 4,
  VT_SGEMM_SKINNY_TF32X3 = 5,
  VT_SGEMM_SKINNY_MMA_SYNC = 6,
  VT_SGEMM_TILE32 = 7,
  VT_SGEMM_PANEL_TF32X3 = 8,
  VT_SGEMM_TALL_TF32X3 = 9,
  VT_SGEMM_PIPE128 = 10,
  VT_SGEMM_PIPE64 = 11,
  VT_SGEMM_PIPE64X128 = 12
};

/* Number of CUDA devices visible, or a negative VT_ERR_* code. */
int vt_device_count(void);

/* Text of the calling thread's last error ("" if none). */
const char* vt_last_error(void);

/* Exact int8 x int8 -> int32 GEMM, C = A(MxK) * B(KxN).
 * Replaces the execution inside run_commands() (specializations/gemmini_gemm/backend.py:433-562,
 * the 16x16x16 compute at :490-529) and scalar_matmul() (:569-580) for streams that compute a
 * full GEMM.  Domain = the reference plan domain (validate_plan, backend.py:107-149): M, N, K >= 16
 * and multiples of 16, K*16384 <= 2^31-1; anything else is VT_ERR_INVALID.  Bit-exact.
 *   raster      VT_RASTER_*;  batch_rows = accumulator_rows/16 for VT_RASTER_BATCHED (else ignored)
 *   variant     VT_I8_* */
int vt_i8gemm(int dev, const int8_t* A, const int8_t* B, int32_t* C, int64_t M, int64_t N, int64_t K, int raster,
              int batch_rows, int variant, int where, void* stream);

/* Batched B-reuse GEMM: `batch` independent A_i (MxK each, stacked contiguously) against one
 * shared B (KxN); C_i (MxN each) stacked likewise.  Replaces executing
 * gen_batched_reuse_b(plan, batch_rows) (specializations/gemmini_gemm/lowering.py:18-40) once per
 * A_i with the same B.  acc_rows is the plan's accumulator_rows (a multiple of 16, 16..1024). */
int vt_i8gemm_shared_b(int dev, const int8_t* A, const int8_t* B, int32_t* C, int64_t batch, int64_t M, int64_t N,
                       int64_t K, int acc_rows, int where, void* stream);

/* One rank's step of a row-sharded int8 GEMM whose replicated operand arrives in pieces: C (M x N) is this rank's
 * row block in HOST memory; A (M x K), its rows of the left operand, is in host memory too (a_where = VT_HOST: the
 * call copies it in first) or already on the device (VT_DEVICE: valid by the time block_ready[0] completes; a
 * caller that queues its own copy of A *before* it stages the blocks of B keeps A from waiting behind them on the
 * host link).  B comes as `n_blocks` column blocks already in this GPU's memory,
 * block j a dense K x block_cols[j] matrix (row pitch block_cols[j]) holding the next block_cols[j] columns of B,
 * valid once the cudaEvent_t block_ready[j] has completed (the caller records it after the broadcast that
 * delivered the block).  The call copies A in, computes the columns of C a block completes as soon as that block
 * is there, returns them to the host while later blocks are still arriving, and returns when C is complete.  Like
 * the row-sharded form of vt_i8gemm it has no counterpart in the reference (which has no multi-device code); it
 * runs the arithmetic of run_commands() (specializations/gemmini_gemm/backend.py:433-562) on this rank's rows.
 * Block widths: multiples of 16, adding up to N; at most 64 blocks. */
int vt_i8gemm_rows_streamed_b(int dev, const int8_t* A, int a_where, const int8_t* const* B_blocks,
                              const int64_t* block_cols, void* const* block_ready, int n_blocks, int32_t* C, int64_t M,
                              int64_t N, int64_t K, int raster, int batch_rows, int variant);

/* Copies columns [c0, c0 + cols) of a row-major K x N int8 matrix in host memory (pinned, for the copy to be
 * asynchronous) into a dense K x cols block in device memory, on `stream`: how the rank that holds B feeds the
 * blocks of vt_i8gemm_rows_streamed_b before it broadcasts them. */
int vt_i8_stage_b_block(int dev, int8_t* dst, const int8_t* B_host, int64_t K, int64_t N, int64_t c0, int64_t cols,
                        void* stream);

/* Tile program: the arithmetic content of an arbitrary, already validated Gemmini command stream.
 * Output tile t (16x16 int32 at element offset c_off[t], row stride ldc) receives
 * sum_{j in [term_begin[t], term_begin[t+1])} Atile(a_off[j]) * Btile(b_off[j]), where a tile is 16x16
 * int8 at an element offset with row stride lda / ldb.  Replaces the compute/mvout part of
 * run_commands() (backend.py:490-553) for streams that are not a plain GEMM.  All arrays are host
 * pointers; A, B, C follow `where`.  VT_ERR_OVERFLOW if a tile has more than 8191 terms. */
int vt_i8_tile_program(int dev, const int8_t* A, int64_t a_elems, const int8_t* B, int64_t b_elems, int32_t* C,
                       int64_t c_elems, int64_t lda, int64_t ldb, int64_t ldc, int64_t n_tiles,
                       const int64_t* c_off, const int64_t* term_begin, const int64_t* a_off,
                       const int64_t* b_off, int where, void* stream);

/* fp32 GEMM, C = A(MxK) * B(KxN), any positive M, N, K.
 * Replaces running the generated `matmul()` of benchmark_matmul() (specializations/cpu_gemm/
 * runner.py:111-190; loop nest emitted by emit_c.py:83-155).  The reference computes in double;
 * this computes in fp32 (relative Frobenius error <= 1e-5 against float64 is the contract). */
int vt_sgemm(int dev, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int variant,
             int where, void* stream);

/* The kernel VT_SGEMM_AUTO picks on `dev` for an M x N x K product of 16-byte-aligned device operands: a
 * VT_SGEMM_* value other than AUTO, or a negative VT_ERR_* code.  Nothing is launched.  It lets a caller that
 * carries a schedule of its own (tile sizes recovered from a loop nest, specializations/cpu_gemm/runner.py:111-190)
 * see what the library would do before overriding it with an explicit variant. */
int vt_sgemm_auto_variant(int dev, int64_t M, int64_t N, int64_t K);

/* The skinny fp32 GEMM (M <= 16, N % 4 == 0, device pointers only) for hosts that must not let this
 * library allocate: it calls no cudaMalloc / cudaFree and no allocating library routine.  It has no
 * counterpart in the reference; it exists for embedders whose own pool (a framework's caching
 * allocator, a serving runtime with a fixed budget) already owns the GPU's memory, where a
 * library-side cudaMalloc can fail or stall a request by synchronising the device.  The K-split
 * partial tiles that vt_sgemm keeps in cudaMalloc'd workspace live here in one fixed
 * VT_SKINNY_STATIC_SCRATCH_BYTES array inside the library image (held by every GPU that loads the
 * library, until exit).  Shapes whose partial tiles need more are refused with VT_ERR_UNSUPPORTED and
 * a message giving both sizes; vt_sgemm serves those.
 *   - The first call on a device looks up the array's device address (with that device current);
 *     make that first call before starting any stream capture.  The calling thread's current device
 *     is the same after the call as before it.
 *   - All calls share the one array: two calls whose kernels can overlap on the GPU (different
 *     streams, no ordering between them) race on it.  Calls on one stream are safe.  Nothing in
 *     the array has to be cleared between calls.
 *   - `stream` is used as given (a cudaStream_t; NULL is the CUDA default stream).  The call only
 *     enqueues; synchronise the stream yourself.  A, B, C are device pointers on `dev`, B and C
 *     16-byte aligned.  Results are bit-identical to vt_sgemm's VT_SGEMM_SKINNY. */
#define VT_SKINNY_STATIC_SCRATCH_BYTES (8u << 20)
int vt_sgemm_skinny_static_scratch(int dev, const float* A, const float* B, float* C, int64_t M, int64_t N,
                                   int64_t K, void* stream);

/* Waits for `stream` (NULL = the library's stream) on `dev` and returns VT_ERR_DEVICE_WAIT if any
 * kernel since the last check gave up on a bounded wait, VT_ERR_CUDA on an asynchronous CUDA error. */
int vt_sync(int dev, void* stream);

/* TEST HOOK, not for production callers (it has no counterpart in the reference).  Every device-side wait of
 * the kernels is bounded; this sets the bound for later launches on `dev` (`wait_limit_cycles` of the SM
 * clock, <= 0 restores the default of about two seconds) and, with `i8_stop_fill` >= 0, makes the odd CTA of
 * every int8 CTA pair stop feeding its operands at that ring fill, so that the waits for them run out, the
 * kernel tears its pipeline down and returns, and vt_sync() reports VT_ERR_DEVICE_WAIT.  -1 turns it off. */
int vt_test_set_wait_hooks(int dev, int64_t wait_limit_cycles, int i8_stop_fill);

/* TEST HOOK.  Launches one small CTA on `stream` that waits, with the bound set above, for a barrier that
 * nothing ever completes; the wait runs out and the kernel records its status and returns. */
int vt_test_expire_wait(int dev, void* stream);

/* TEST HOOK.  The FFMA tile kernels (VT_SGEMM_TILE128 / TILE64 / TILE32) split K over several CTAs per output
 * tile when the tile grid alone would leave most of the GPU idle.  `splits` > 0 forces that many for later calls
 * on `dev` (as far as K allows, at most 16; the 128- and 64-wide kernels exchange up to 8 partial tiles through
 * the shared memory of a thread-block cluster and more through scratch memory), `splits` < 0 forces -splits
 * through scratch memory, 0 restores the automatic choice.  Results are bit-identical from call to call for a
 * given split (partial tiles are added in split order). */
int vt_test_set_sgemm_splits(int dev, int splits);

/* Pinned host memory for VT_HOST calls. */
void* vt_host_alloc(size_t bytes);
int vt_host_free(void* p);

/* Number of kernels this library has launched in this process (all devices, all threads). */
int64_t vt_launch_count(void);

/* Frees every device context (streams, workspace).  Safe to call more than once. */
int vt_shutdown(void);

#ifdef __cplusplus
}
#endif
#endif /* VERITAC_B200_H */
