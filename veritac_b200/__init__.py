"""veritac_b200 — B200 (sm_100a) execution back end for VeriTac's CodeGen GEMM hot path.

Layout
  csrc/ + libveritac_b200.so   hand-written CUDA kernels behind the C ABI of include/veritac_b200.h
  _native.py                   ctypes binding of that ABI (no CPU fallback)
  specializations/             the reference's `specializations.cpu_gemm` / `.gemmini_gemm` modules
                               re-implemented on top of it; `catalog` lists them
  CodeGen/                     the reference's older import paths, aliased to the same modules
  sharding.py                  row / batch sharding of a GEMM over the ranks of a torch.distributed job

`install_aliases()` makes the reference's top-level names importable (`from CodeGen.runner import
benchmark_matmul`, `from specializations import catalog`), which is all a caller of the reference
has to change.
"""
from __future__ import annotations

import importlib
import sys

__version__ = "0.1.0"


def install_aliases(force: bool = False) -> None:
    """Register `CodeGen` and `specializations` as top-level aliases of this package's sub-packages.

    Refuses (ImportError) to shadow different modules already imported under those names unless
    `force` is given.
    """
    for name in ("specializations", "CodeGen"):
        mod = importlib.import_module(__name__ + "." + name)
        present = sys.modules.get(name)
        if present is not None and present is not mod and not force:
            raise ImportError("a different top-level module %r is already imported" % name)
        sys.modules[name] = mod
    for sub, leaves in (("cpu_gemm", ("lower", "emit_c", "runner", "recognise")),
                        ("gemmini_gemm", ("backend", "lowering", "evaluation", "schedule_ir"))):
        sys.modules["specializations." + sub] = importlib.import_module(__name__ + ".specializations." + sub)
        for leaf in leaves:    # one module object per file, whichever name it is imported under
            sys.modules["specializations.%s.%s" % (sub, leaf)] = importlib.import_module(
                "%s.specializations.%s.%s" % (__name__, sub, leaf))
    sys.modules["specializations.catalog"] = importlib.import_module(__name__ + ".specializations.catalog")
