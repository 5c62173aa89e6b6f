"""The multi-rank host logic on CPU: two gloo ranks shard M by rows, rank 0's B is replicated by a
broadcast, each rank computes only its block (the exact CPU product stands in for the device call),
and the assembled C equals the unsharded product."""
import os
import subprocess
import sys

import pytest

from conftest import REPO
from veritac_b200.sharding import batch_shard, column_blocks, row_shard


def test_row_shard_tiles_the_range():
    for rows in (0, 16, 48, 8192, 8192 * 8, 1040):
        for world in (1, 2, 3, 4, 8):
            spans = [row_shard(rows, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == rows
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0
            sizes = [e - b for b, e in spans]
            assert all(s % 16 == 0 for s in sizes) and max(sizes) - min(sizes) <= 16
    assert [row_shard(8192, 8, r) for r in (0, 7)] == [(0, 1024), (7168, 8192)]
    assert [batch_shard(256, 8, r) for r in (0, 1, 7)] == [(0, 32), (32, 64), (224, 256)]
    with pytest.raises(ValueError):
        row_shard(100, 2, 0)
    with pytest.raises(ValueError):
        row_shard(64, 2, 2)


def test_column_blocks_tile_the_columns():
    for n in (16, 256, 272, 4096, 8192, 8192 + 48, 1000 * 16):
        for nb in (1, 2, 3, 8, 64):
            blocks = column_blocks(n, nb)
            assert blocks[0][0] == 0 and sum(c for _, c in blocks) == n and len(blocks) <= nb
            for (a0, ac), (b0, _bc) in zip(blocks, blocks[1:]):
                assert a0 + ac == b0
            assert all(c % 256 == 0 for _, c in blocks[:-1]) and all(c > 0 for _, c in blocks)
    assert column_blocks(8192, 8) == [(i * 1024, 1024) for i in range(8)]
    with pytest.raises(ValueError):
        column_blocks(0, 4)


WORKER = r"""
import os, sys
sys.path.insert(0, {repo!r}); sys.path.insert(0, {repo!r} + "/oracle")
import numpy as np, torch, torch.distributed as dist
from veritac_b200 import sharding
import gemmini_oracle as go
rank, world, _ = sharding.init_process_group(backend="gloo", timeout_s=60)
M, N, K = 80, 48, 64
rng = np.random.default_rng(123)
A = rng.integers(-128, 128, (M, K), dtype=np.int8)             # every rank can regenerate A ...
B_true = rng.integers(-128, 128, (K, N), dtype=np.int8)
B_source = torch.from_numpy(B_true.copy()) if rank == 0 else None   # ... but B exists on rank 0 only
B = torch.zeros((K, N), dtype=torch.int8)
r0, r1 = sharding.row_shard(M, world, rank)
C_rows = np.full((r1 - r0, N), -2**31, dtype=np.int32)
def compute(a, b, c):
    c[:] = go.matmul_exact(a, b.numpy(), a.shape[0], N, K).astype(np.int32)
sharding.run_row_sharded(compute, A[r0:r1], B, C_rows, B_source=B_source)
assert np.array_equal(B.numpy(), B_true)                         # it arrived by the broadcast
# the same step with B delivered in column blocks: rank 0 stages each block, the broadcast carries it on
blocks = sharding.column_blocks(N, 2, align=16)
bufs = [torch.zeros((K, cols), dtype=torch.int8) for _c0, cols in blocks]
C2 = np.full((r1 - r0, N), -2**31, dtype=np.int32)
staged = []
def stage(j, buf, c0, cols):
    staged.append(j)
    buf.copy_(torch.from_numpy(B_true[:, c0:c0 + cols].copy()))
def compute_blocks(a, bs, markers, c):
    assert markers == ["ready0", "ready1"]
    c[:] = go.matmul_exact(a, np.concatenate([b.numpy() for b in bs], axis=1), a.shape[0], N, K).astype(np.int32)
sharding.run_row_sharded_streamed(stage, compute_blocks, A[r0:r1], bufs, C2, blocks, mark_ready=lambda j: "ready%d" % j)
assert staged == ([0, 1] if rank == 0 else []) and np.array_equal(C2, C_rows)
parts = [None] * world
dist.all_gather_object(parts, (r0, r1, C_rows))
C = np.concatenate([p[2] for p in sorted(parts, key=lambda p: p[0])])
assert np.array_equal(C, go.matmul_exact(A, B_true, M, N, K).astype(np.int32))
assert sorted((p[0], p[1]) for p in parts) == [(0, 48), (48, 80)]
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_two_rank_gloo_row_sharding(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(repo=str(REPO)))
    port = 29500 + (os.getpid() % 2000)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "rank %d ok" % rank in out, out
