"""TEST INFRASTRUCTURE — builds the C restatements under cref/ into oracle/liboracle.so.

Picks the first C compiler that can compile *and link* an OpenMP program, trying VERITAC_CC first
and then the same candidates the reference's runner tries (specializations/cpu_gemm/runner.py:42-62).
`python oracle/build_oracle.py` prints the library path.
"""
from __future__ import annotations

import os
import subprocess
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "liboracle.so"
SOURCES = [HERE / "cref" / "i8gemm_ref.c", HERE / "cref" / "fgemm_ref.c"]


def find_openmp_cc():
    cands = [os.environ.get("VERITAC_CC"), "gcc-16", "gcc-15", "gcc-14", "gcc-13", "gcc-12", "/usr/bin/gcc", "gcc",
             "cc", "clang"]
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "probe.c")
        with open(src, "w") as fh:
            fh.write("#include <omp.h>\nint main(void){return omp_get_max_threads() < 1;}\n")
        for cc in cands:
            if not cc:
                continue
            try:
                r = subprocess.run([cc, "-fopenmp", "-O2", "-o", os.path.join(tmp, "probe"), src],
                                   capture_output=True, text=True, timeout=30)
            except (FileNotFoundError, subprocess.TimeoutExpired):
                continue
            if r.returncode == 0:
                return cc
    return None


def build(force=False):
    if not force and LIB.is_file() and all(LIB.stat().st_mtime >= s.stat().st_mtime for s in SOURCES):
        return LIB
    cc = find_openmp_cc()
    if cc is None:
        raise RuntimeError("no OpenMP-capable C compiler found")
    cmd = [cc, "-O2", "-fopenmp", "-fPIC", "-Wall", "-shared", "-o", str(LIB)] + [str(s) for s in SOURCES]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
