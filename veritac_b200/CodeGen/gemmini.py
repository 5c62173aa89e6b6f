"""Compatibility entry point: this module *is* specializations.gemmini_gemm.backend (same module object),
as in the reference's CodeGen/gemmini.py:1-9."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module(
    __name__.rsplit(".CodeGen.", 1)[0] + ".specializations.gemmini_gemm.backend" if ".CodeGen." in __name__
    else "specializations.gemmini_gemm.backend")
