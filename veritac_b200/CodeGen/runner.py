"""Compatibility entry point: this module *is* specializations.cpu_gemm.runner (same module object),
as in the reference's CodeGen/runner.py:1-9."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module(
    __name__.rsplit(".CodeGen.", 1)[0] + ".specializations.cpu_gemm.runner" if ".CodeGen." in __name__
    else "specializations.cpu_gemm.runner")
