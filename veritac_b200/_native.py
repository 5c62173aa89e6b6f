"""ctypes binding of libveritac_b200.so (the C ABI in include/veritac_b200.h).

There is no CPU fallback: if the shared library is missing or a call fails, a `NativeError` is
raised.  The library is built in-tree by `python -m veritac_b200.build`.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libveritac_b200.so"

VT_OK = 0
VT_ERR_INVALID = -1
VT_ERR_CUDA = -2
VT_ERR_DEVICE_WAIT = -3
VT_ERR_UNSUPPORTED = -4
VT_ERR_OVERFLOW = -5
VT_ERR_PROGRAM = -6

VT_HOST = 0
VT_DEVICE = 1
VT_HOST_AC_DEVICE_B = 2

VT_RASTER_BASELINE = 0
VT_RASTER_REUSE_B = 1
VT_RASTER_BATCHED = 2
VT_RASTER_AUTO = 3

VT_I8_AUTO = 0
VT_I8_B_AS_STORED = 1
VT_I8_CTA_PAIR = 3
VT_I8_CTA_PAIR_WIDE = 4

VT_SGEMM_AUTO = 0
VT_SGEMM_TILE128 = 1
VT_SGEMM_TILE64 = 2
VT_SGEMM_SKINNY = 3
VT_SGEMM_TF32X3 = 4
VT_SGEMM_SKINNY_TF32X3 = 5
VT_SGEMM_SKINNY_MMA_SYNC = 6
VT_SGEMM_TILE32 = 7
VT_SGEMM_PANEL_TF32X3 = 8
VT_SGEMM_TALL_TF32X3 = 9
VT_SGEMM_PIPE128 = 10
VT_SGEMM_PIPE64 = 11
VT_SGEMM_PIPE64X128 = 12

SGEMM_VARIANT_NAMES = {0: "AUTO", 1: "TILE128", 2: "TILE64", 3: "SKINNY", 4: "TF32X3", 5: "SKINNY_TF32X3",
                       6: "SKINNY_MMA_SYNC", 7: "TILE32", 8: "PANEL_TF32X3", 9: "TALL_TF32X3",
                       10: "PIPE128", 11: "PIPE64", 12: "PIPE64X128"}

# Every symbol include/veritac_b200.h declares, with its ctypes signature.
SIGNATURES = {
    "vt_device_count": (c_int, []),
    "vt_last_error": (c_char_p, []),
    "vt_i8gemm": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_int,
                          c_int, c_void_p]),
    "vt_i8gemm_shared_b": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int,
                                   c_int, c_void_p]),
    "vt_i8gemm_rows_streamed_b": (c_int, [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64,
                                          c_int64, c_int64, c_int, c_int, c_int]),
    "vt_i8_stage_b_block": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "vt_i8_tile_program": (c_int, [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64,
                                   c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "vt_sgemm": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_void_p]),
    "vt_sgemm_auto_variant": (c_int, [c_int, c_int64, c_int64, c_int64]),
    "vt_sgemm_skinny_static_scratch": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                               c_void_p]),
    "vt_test_set_wait_hooks": (c_int, [c_int, c_int64, c_int]),
    "vt_test_set_sgemm_splits": (c_int, [c_int, c_int]),
    "vt_test_expire_wait": (c_int, [c_int, c_void_p]),
    "vt_sync": (c_int, [c_int, c_void_p]),
    "vt_host_alloc": (c_void_p, [c_size_t]),
    "vt_host_free": (c_int, [c_void_p]),
    "vt_launch_count": (c_int64, []),
    "vt_shutdown": (c_int, []),
}


class NativeError(RuntimeError):
    """A C-ABI call failed; `.code` is the VT_ERR_* value."""

    def __init__(self, code: int, message: str):
        super().__init__("veritac_b200 native call failed (%d): %s" % (code, message))
        self.code = code
        self.message = message


_lib = None


def lib() -> ctypes.CDLL:
    """The loaded shared library; raises NativeError if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.is_file():
            raise NativeError(VT_ERR_UNSUPPORTED,
                              "%s is missing: run `python -m veritac_b200.build` (there is no CPU fallback)"
                              % LIB_PATH)
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def last_error() -> str:
    return (lib().vt_last_error() or b"").decode("utf-8", "replace")


def check(code: int) -> int:
    if code < 0:
        raise NativeError(code, last_error())
    return code


def device_count() -> int:
    return check(lib().vt_device_count())


def launch_count() -> int:
    return int(lib().vt_launch_count())


def _ptr(x) -> int:
    """Address of a numpy array's or torch tensor's first element."""
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    if hasattr(x, "ctypes"):
        return int(x.ctypes.data)
    return int(x)


def torch_stream() -> int:
    """Handle of torch's current CUDA stream in the form the C ABI takes.

    The ABI reads NULL as "the library's own stream", so torch's legacy default stream (handle 0)
    is passed as cudaStreamLegacy (0x1).
    """
    import torch

    return int(torch.cuda.current_stream().cuda_stream) or 1


def i8gemm(A, B, C, M: int, N: int, K: int, *, dev: int = 0, raster: int = VT_RASTER_AUTO, batch_rows: int = 1,
           variant: int = VT_I8_AUTO, where: int = VT_HOST, stream: int = 0) -> None:
    check(lib().vt_i8gemm(dev, _ptr(A), _ptr(B), _ptr(C), M, N, K, raster, batch_rows, variant, where, stream))


def i8gemm_shared_b(A, B, C, batch: int, M: int, N: int, K: int, *, dev: int = 0, acc_rows: int = 16,
                    where: int = VT_HOST, stream: int = 0) -> None:
    check(lib().vt_i8gemm_shared_b(dev, _ptr(A), _ptr(B), _ptr(C), batch, M, N, K, acc_rows, where, stream))


def i8_stage_b_block(dst, B_host, K: int, N: int, c0: int, cols: int, *, dev: int = 0, stream: int = 0) -> None:
    """Columns [c0, c0 + cols) of the row-major host matrix B into the dense device block `dst`, asynchronously."""
    check(lib().vt_i8_stage_b_block(dev, _ptr(dst), _ptr(B_host), K, N, c0, cols, stream))


def i8gemm_rows_streamed_b(A, B_blocks, block_cols, block_ready, C, M: int, N: int, K: int, *, dev: int = 0,
                           a_where: int = VT_HOST, raster: int = VT_RASTER_AUTO, batch_rows: int = 1,
                           variant: int = VT_I8_AUTO) -> None:
    """One rank's rows of an int8 GEMM with B arriving in column blocks (see the header).  `B_blocks` are device
    tensors or pointers, `block_ready` CUDA event handles (torch.cuda.Event.cuda_event or integers); `a_where`
    says whether A is a host buffer the call copies in or already on the device."""
    n = len(B_blocks)
    ptrs = (c_void_p * n)(*[_ptr(b) for b in B_blocks])
    cols = (c_int64 * n)(*[int(x) for x in block_cols])
    evs = (c_void_p * n)(*[int(getattr(e, "cuda_event", e)) for e in block_ready])
    check(lib().vt_i8gemm_rows_streamed_b(dev, _ptr(A), a_where, ptrs, cols, evs, n, _ptr(C), M, N, K, raster, batch_rows,
                                          variant))


def i8_tile_program(A, a_elems, B, b_elems, C, c_elems, lda, ldb, ldc, c_off, term_begin, a_off, b_off, *,
                    dev: int = 0, where: int = VT_HOST, stream: int = 0) -> None:
    n_tiles = len(c_off)
    check(lib().vt_i8_tile_program(dev, _ptr(A), a_elems, _ptr(B), b_elems, _ptr(C), c_elems, lda, ldb, ldc,
                                   n_tiles, _ptr(c_off), _ptr(term_begin), _ptr(a_off), _ptr(b_off), where, stream))


def sgemm(A, B, C, M: int, N: int, K: int, *, dev: int = 0, variant: int = VT_SGEMM_AUTO, where: int = VT_HOST,
          stream: int = 0) -> None:
    check(lib().vt_sgemm(dev, _ptr(A), _ptr(B), _ptr(C), M, N, K, variant, where, stream))


def sgemm_auto_variant(M: int, N: int, K: int, *, dev: int = 0) -> int:
    """The VT_SGEMM_* kernel the automatic choice takes for this shape (aligned device operands)."""
    return check(lib().vt_sgemm_auto_variant(dev, M, N, K))


SKINNY_STATIC_SCRATCH_BYTES = 8 << 20


def sgemm_skinny_static_scratch(A, B, C, M: int, N: int, K: int, *, dev: int = 0, stream: int = 0) -> None:
    """Skinny fp32 GEMM on device pointers that allocates nothing (see the header for the limits)."""
    check(lib().vt_sgemm_skinny_static_scratch(dev, _ptr(A), _ptr(B), _ptr(C), M, N, K, stream))


def test_set_wait_hooks(dev: int = 0, wait_limit_cycles: int = 0, i8_stop_fill: int = -1) -> None:
    """Test hook: bound of the device-side waits (0 = default) and the int8 pair kernel's induced stop."""
    check(lib().vt_test_set_wait_hooks(dev, wait_limit_cycles, i8_stop_fill))


def test_set_sgemm_splits(splits: int = 0, dev: int = 0) -> None:
    """Test hook: K split of the FFMA tile kernels (0 = automatic)."""
    check(lib().vt_test_set_sgemm_splits(dev, splits))


def test_expire_wait(dev: int = 0, stream: int = 0) -> None:
    """Test hook: enqueue one CTA whose bounded wait runs out."""
    check(lib().vt_test_expire_wait(dev, stream))


def sync(dev: int = 0, stream: int = 0) -> None:
    check(lib().vt_sync(dev, stream))


def shutdown() -> None:
    check(lib().vt_shutdown())
