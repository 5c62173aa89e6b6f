"""The reference arm of bench.py (the CPU leg, no GPU needed): one JSON line with the agreed keys."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent


def run_reference_arm(workload):
    r = subprocess.run([sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--workload", workload,
                        "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=300, cwd=REPO)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [x for x in r.stdout.splitlines() if x.startswith("{")]
    assert len(lines) == 1
    return json.loads(lines[0])


@pytest.mark.parametrize("workload", ["i8_64", "sgemm_256"])
def test_reference_arm_line(workload):
    line = run_reference_arm(workload)
    assert line["impl"] == "reference" and line["value"] > 0 and line["higher_is_better"] is True
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["warmup"] == 0 and line["gpu_launches"] == 0
    cpu = line["cpu_baseline"]
    assert cpu["value"] == line["value"] and cpu["cores"] >= 1 and cpu["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    if workload == "sgemm_256" and (REPO / "oracle" / "_ref" / "matmul_256_readme.so").is_file():
        assert cpu["kind"] == "reference"       # the reference's own generated C, built ahead of time
    else:
        assert cpu["kind"] == "port"
