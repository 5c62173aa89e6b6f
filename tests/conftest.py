"""Shared test configuration.

`-m "not gpu"` tests need no CUDA device: they cover the oracle against the reference's golden
vectors, the host-side logic, and that the C-ABI library loads and exports what the header declares.
`-m gpu` tests are the parity tests proper and call the CUDA path through the C ABI.
"""
import json
import os
import stat
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]
GOLDEN = REPO / "tests" / "golden"
STUB = REPO / "oracle" / "gemmini_check_stub.py"

for p in (str(REPO), str(REPO / "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)

# The Lean plan checker is not part of this build; the reference's documented override points at
# the oracle's restatement of it so that run_commands can pass its fail-closed gate in tests.
if not os.access(STUB, os.X_OK):
    os.chmod(STUB, os.stat(STUB).st_mode | stat.S_IXUSR | stat.S_IXGRP | stat.S_IXOTH)
os.environ["VERITAC_GEMMINI_CHECK_BIN"] = str(STUB)
# Likewise the tactic verifier (`veritac --json`): the demo that drives it takes the executable's path from
# VERITAC_BIN, which tests point at the oracle's restatement of the four tactics.
CLI_STUB = REPO / "oracle" / "veritac_cli_stub.py"
if not os.access(CLI_STUB, os.X_OK):
    os.chmod(CLI_STUB, os.stat(CLI_STUB).st_mode | stat.S_IXUSR | stat.S_IXGRP | stat.S_IXOTH)
os.environ["VERITAC_BIN"] = str(CLI_STUB)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden_gemmini():
    return json.loads((GOLDEN / "gemmini.json").read_text())


@pytest.fixture(scope="session")
def golden_schedule_ir():
    return json.loads((GOLDEN / "schedule_ir.json").read_text())


@pytest.fixture(scope="session")
def golden_learned_streams():
    return json.loads((GOLDEN / "learned_streams.json").read_text())


@pytest.fixture(scope="session")
def golden_cpu_gemm():
    return json.loads((GOLDEN / "cpu_gemm.json").read_text())


@pytest.fixture(scope="session")
def native():
    """The ctypes binding with the library built (nvcc cross-compiles without a GPU)."""
    from veritac_b200 import build

    build.build()
    from veritac_b200 import _native

    _native.lib()
    return _native


@pytest.fixture(scope="session")
def liboracle():
    """ctypes handle of the C restatements under oracle/cref."""
    import ctypes

    import build_oracle

    lib = ctypes.CDLL(str(build_oracle.build()))
    i64, vp = ctypes.c_long, ctypes.c_void_p
    lib.oracle_i8_scalar_ref.argtypes = [vp, vp, vp, i64, i64, i64]
    lib.oracle_i8_tiled_ref.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64]
    lib.oracle_i8_lcg_inputs.argtypes = [vp, i64, vp, i64, ctypes.c_uint32]
    for name in ("oracle_dgemm_naive", "oracle_sgemm_naive", "oracle_dgemm_tuned", "oracle_sgemm_tuned"):
        getattr(lib, name).argtypes = [vp, vp, vp, i64, i64, i64]
    return lib


class Cmd:
    """A command object rebuilt from its serialized dict (the form fixtures store)."""

    def __init__(self, d):
        self.__dict__.update({k: v for k, v in d.items() if k != "kind"})
        self.kind = d["kind"]


def commands_from_dicts(dicts):
    return [Cmd(d) for d in dicts]
