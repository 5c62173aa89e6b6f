"""Compatibility entry point: this module *is* specializations.cpu_gemm.emit_c (same module object),
as in the reference's CodeGen/emit_c.py:1-9."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module(
    __name__.rsplit(".CodeGen.", 1)[0] + ".specializations.cpu_gemm.emit_c" if ".CodeGen." in __name__
    else "specializations.cpu_gemm.emit_c")
