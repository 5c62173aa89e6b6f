"""The row-sharded job on two real GPUs (skipped where fewer are visible): `bench.py --gpus 2` under torchrun, one
short run.  Every rank checks sampled rows of its C against the exact product, for the device-resident run and for
the end-to-end run whose B crosses the host link on rank 0 only and reaches the other GPU by NCCL broadcast in
column blocks; the line must say so, carry the split shape, and report the broadcast apart from the communicator's
creation.  The other workloads of the line run as well, so that a rank that drifts to another rank's GPU shows."""
import json
import os
import subprocess
import sys

import pytest

from conftest import REPO

pytestmark = pytest.mark.gpu


def test_two_rank_bench_line_and_parity():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = 29600 + (os.getpid() % 300)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(REPO / "bench.py"), "--gpus", "2",
                        "--steps", "3", "--warmup", "3", "--sustain-seconds", "0"],
                       capture_output=True, text=True, timeout=600, cwd=REPO, env=env)
    assert r.returncode == 0, r.stderr[-3000:]
    lines = [x for x in r.stdout.splitlines() if x.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["n_gpus"] == 2 and line["scaling"] == "strong"
    assert line["config"]["global_M"] == 8192 and line["config"]["M_per_gpu"] == 4096
    assert line["parity"]["ok"] is True and line["parity"]["ranks"] == 2
    assert line["parity"]["host_buffer_run"]["cells_differing"] == 0
    assert line["config"]["bcast_ms_warm"] < 50 < line["config"]["comm_init_ms"]
    assert "rank 0 only" in line["e2e"]["bytes"] and line["e2e"]["link_floor_ms"] > 0
    assert line["gpu_launches"] == 3 and line["value"] > 0
    # the other workloads ran on both ranks too (rank 1 on its own GPU) and every one checked its result
    assert set(line["also"]) >= {"sgemm_8192", "sgemm_8192_ffma", "sgemm_skinny", "i8_batched", "sgemm_256", "sgemm_640"}
    assert all(v["parity_ok"] for v in line["also"].values())
    assert line["weak"]["parity_ok"] is True


def test_a_question_about_another_gpu_leaves_the_current_device_alone(native):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    torch.cuda.set_device(0)
    assert native.sgemm_auto_variant(640, 640, 640, dev=1) > 0
    assert torch.cuda.current_device() == 0
    assert torch.empty(1, device="cuda").device.index == 0
