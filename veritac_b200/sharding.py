"""Sharding one GEMM over the GPUs of a box: one process per GPU, torch.distributed for plumbing.

Every output row of C = A * B depends on one row of A and all of B (the reference's spec:
VeriTac/Gemmini/Semantics.lean:76-77), so the path shards with no reduction: rank r owns a block of
rows of A and C (or a block of the batch for the shared-B form) and B is replicated — broadcast once
from rank 0 into each GPU's own HBM, outside the steady state.  Kernels only ever read local memory;
there is no data-path collective and no split-K.
"""
from __future__ import annotations

import os


def row_shard(rows: int, world: int, rank: int, align: int = 16) -> tuple[int, int]:
    """[begin, end) of the rows rank `rank` of `world` owns.

    Blocks are contiguous, multiples of `align` (16 keeps every shard inside the Gemmini plan
    domain), differ by at most one `align` block, and tile [0, rows) exactly.  `rows` itself must be
    a multiple of `align`.  A rank may get an empty block when there are fewer blocks than ranks.
    """
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank %d outside world of %d" % (rank, world))
    if rows < 0 or rows % align:
        raise ValueError("rows=%d must be a non-negative multiple of %d" % (rows, align))
    blocks = rows // align
    base, extra = divmod(blocks, world)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return begin * align, end * align


def batch_shard(batch: int, world: int, rank: int) -> tuple[int, int]:
    """[begin, end) of the batch entries (independent A_i against one shared B) a rank owns."""
    return row_shard(batch, world, rank, align=1)


def env_rank() -> tuple[int, int, int]:
    """(rank, world_size, local_rank) from the torchrun environment; (0, 1, 0) outside it."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def init_process_group(backend: str | None = None, timeout_s: float = 120.0):
    """Joins the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT.

    `backend` defaults to nccl when CUDA is available, else gloo.  Returns (rank, world, local_rank);
    with WORLD_SIZE 1 no process group is created.
    """
    import datetime

    import torch
    import torch.distributed as dist

    rank, world, local = env_rank()
    if world == 1:
        return rank, world, local
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if not dist.is_initialized():
        extra = {"device_id": torch.device("cuda", local)} if backend == "nccl" else {}
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **extra)
    return rank, world, local


def replicate_from_rank0(tensor):
    """Broadcast `tensor` (B) from rank 0 into every rank's own memory; returns it.  A single-rank
    job returns the tensor untouched."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.broadcast(tensor, src=0)
    return tensor


def run_row_sharded(compute, A_rows, B_local, C_rows, B_source=None):
    """One end-to-end step of the row-sharded product on this rank.

    `B_source` is the job's B where it originates, on rank 0 only (a pinned host tensor in the GPU job): rank 0
    copies it into its `B_local`, the broadcast then delivers it into every other rank's `B_local` over the
    GPU interconnect, so B crosses the host link once per job step instead of once per rank.  After that
    `compute(A_rows, B_local, C_rows)` runs on this rank's block (for int8: `_native.i8gemm` with
    VT_HOST_AC_DEVICE_B, which copies the block of A in and the block of C out); a rank with an empty block
    still takes part in the broadcast.  The same function drives the CPU test, where `compute` is a checker.
    """
    import torch.distributed as dist

    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    if B_source is not None and rank == 0:
        B_local.copy_(B_source, non_blocking=True)
    replicate_from_rank0(B_local)
    if A_rows.shape[0] > 0:
        compute(A_rows, B_local, C_rows)
    return C_rows


def column_blocks(N: int, n_blocks: int, align: int = 256) -> list[tuple[int, int]]:
    """[(first column, width)] of at most `n_blocks` blocks that tile [0, N): widths are multiples of `align`
    (the int8 kernels' tile width) except possibly the last, and differ by at most one `align`."""
    if N <= 0 or n_blocks < 1:
        raise ValueError("N and n_blocks must be positive")
    units = -(-N // align)
    n_blocks = min(n_blocks, units)
    base, extra = divmod(units, n_blocks)
    out, c0 = [], 0
    for j in range(n_blocks):
        cols = min((base + (1 if j < extra else 0)) * align, N - c0)
        out.append((c0, cols))
        c0 += cols
    return out


def run_row_sharded_streamed(stage_block, compute, A_rows, B_blocks, C_rows, blocks, mark_ready=None):
    """The row-sharded step with B delivered in column blocks, so that a rank starts computing (and returning C)
    while later blocks of B are still on the host link or the interconnect.

    `blocks` is column_blocks(N, ...); `B_blocks[j]` is this rank's buffer for block j (a dense K x cols tensor).
    On rank 0 `stage_block(j, B_blocks[j], c0, cols)` fills the buffer from wherever B originates (for the GPU job:
    `_native.i8_stage_b_block` from pinned host memory); every block is then broadcast from rank 0, and
    `mark_ready(j)` (for the GPU job: record a CUDA event after the broadcast) yields the marker the compute call
    waits on.  `compute(A_rows, B_blocks, markers, C_rows)` runs once, after all blocks have been *queued*: on a GPU
    the copies and broadcasts are asynchronous, so the call (`_native.i8gemm_rows_streamed_b`) overlaps them.
    """
    import torch.distributed as dist

    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    markers = []
    for j, (c0, cols) in enumerate(blocks):
        if rank == 0:
            stage_block(j, B_blocks[j], c0, cols)
        replicate_from_rank0(B_blocks[j])
        markers.append(mark_ready(j) if mark_ready is not None else None)
    if A_rows.shape[0] > 0:
        compute(A_rows, B_blocks, markers, C_rows)
    return C_rows
