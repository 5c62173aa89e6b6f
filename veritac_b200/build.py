"""Builds the in-tree shared library `veritac_b200/libveritac_b200.so` for sm_100a with nvcc.

Run as `python -m veritac_b200.build` (add `--force` to rebuild, `--verbose` for ptxas resource
usage).  The library is a plain C-ABI shared object (see include/veritac_b200.h); nothing in it
depends on Python or torch.  nvcc cross-compiles, so this works on a machine without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libveritac_b200.so"
SOURCES = ["runtime.cu", "i8gemm_sm100.cu", "i8gemm_wide_sm100.cu", "i8_tileprog.cu", "sgemm_sm100.cu", "sgemm_ffma_sm100.cu", "sgemm_tf32x3_sm100.cu",
           "sgemm_skinny_tma_sm100.cu", "sgemm_skinny_umma_sm100.cu", "capi.cu"]
HEADERS = ["runtime.h", "ptx_sm100.cuh", "umma_tile.cuh", "skinny_sched.cuh", "../../include/veritac_b200.h"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def _stale() -> bool:
    if not LIB.is_file():
        return True
    built = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + [(CSRC / h).resolve() for h in HEADERS] + [Path(__file__)]
    return any(d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu under csrc/ into one shared object next to this file."""
    if not force and not _stale():
        return LIB
    nvcc = _nvcc()
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    common = [nvcc, *ARCH, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    objs = []
    for src in SOURCES:
        obj = objdir / (Path(src).stem + ".o")
        objs.append(str(obj))
        procs.append((src, subprocess.Popen(common + ["-c", str(CSRC / src), "-o", str(obj)],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = []
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            failed.append(src)
    if failed:
        raise RuntimeError("nvcc failed for: " + ", ".join(failed))
    link = [nvcc, *ARCH, "-shared", "-o", str(LIB), *objs]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
