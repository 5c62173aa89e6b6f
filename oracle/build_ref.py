"""TEST INFRASTRUCTURE — builds artefacts of the *reference itself* into oracle/_ref/ (git-ignored).

The reference's cpu_gemm path is a Python emitter whose product is generated OpenMP C.  Where the
reference tree is present (the directory REFERENCE_ROOT names, else a directory `reference` beside this
repository) this script imports its
unmodified emitter (CodeGen/emit_c.py, CodeGen/lower.py), has it print `matmul()` for the 256^3 nest —
untuned, and after the schedule its README quotes (tactics applied by oracle/loopnest_oracle.py,
because the Lean CLI that applies them cannot be built here) — and compiles each text to a shared
object exporting `matmul(const double* A, const double* B, double* C)` in the reference's 1000-stride
layout.  Nothing of the reference's sources is copied into the repository; only these outputs land
in oracle/_ref/.  Without the reference tree the script does nothing and says so.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
REF = Path(os.environ.get("REFERENCE_ROOT") or HERE.parents[1] / "reference")
SHAPES = [(256, 256, 256), (512, 512, 512)]


def build() -> list[Path]:
    if not (REF / "CodeGen" / "emit_c.py").is_file():
        print("reference tree not found at %s; nothing built" % REF)
        return []
    sys.dont_write_bytecode = True
    sys.path.insert(0, str(HERE))
    import build_oracle
    import loopnest_oracle as lo

    saved = list(sys.path)
    sys.path.insert(0, str(REF))
    try:
        from CodeGen import emit_c as ref_emit
        from CodeGen import lower as ref_lower
    finally:
        sys.path[:] = saved
    cc = build_oracle.find_openmp_cc()
    if cc is None:
        raise RuntimeError("no OpenMP-capable C compiler found")
    OUT.mkdir(exist_ok=True)
    built = []
    for (M, K, N) in SHAPES:
        for tag, tactics in (("naive", []), ("readme", lo.README_SCHEDULE)):
            stmt = lo.apply_tactics(lo.matmul_stmt(M, K, N), tactics)
            text = ref_emit.emit_function("matmul", ref_lower.parse_stmt(stmt), [("A", 0), ("B", 0)], [("C", 0)])
            src = OUT / ("matmul_%d_%s.c" % (M, tag))
            lib = OUT / ("matmul_%d_%s.so" % (M, tag))
            src.write_text(text)
            r = subprocess.run([cc, "-fopenmp", "-O2", "-fPIC", "-shared", "-o", str(lib), str(src), "-lm"],
                               capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError("compiling %s failed:\n%s" % (src, r.stderr))
            built.append(lib)
    return built


if __name__ == "__main__":
    for p in build():
        print(p)
