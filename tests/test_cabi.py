"""The C-ABI shared library: it builds, loads, exports exactly what include/veritac_b200.h
declares, and rejects out-of-domain arguments before touching a device.  No compute calls."""
import ctypes
import re

import pytest

from conftest import REPO


def declared_symbols():
    text = (REPO / "include" / "veritac_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vt_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(native):
    names = declared_symbols()
    assert names == sorted(native.SIGNATURES), "ctypes table and header differ"
    handle = ctypes.CDLL(str(native.LIB_PATH))
    for name in names:
        assert hasattr(handle, name), name
    assert len(names) == 18


def test_status_codes_match_header(native):
    text = (REPO / "include" / "veritac_b200.h").read_text()
    for name in ("VT_OK", "VT_ERR_INVALID", "VT_ERR_CUDA", "VT_ERR_DEVICE_WAIT", "VT_ERR_UNSUPPORTED",
                 "VT_ERR_OVERFLOW", "VT_ERR_PROGRAM"):
        m = re.search(r"\b%s\s*=\s*(-?\d+)" % name, text)
        assert m and int(m.group(1)) == getattr(native, name)
    for group in ("VT_RASTER_BASELINE|VT_RASTER_REUSE_B|VT_RASTER_BATCHED|VT_RASTER_AUTO",
                  "VT_I8_AUTO|VT_I8_B_AS_STORED|VT_I8_CTA_PAIR|VT_I8_CTA_PAIR_WIDE",
                  "VT_SGEMM_AUTO|VT_SGEMM_TILE128|VT_SGEMM_TILE64|VT_SGEMM_SKINNY|VT_SGEMM_TF32X3|VT_SGEMM_SKINNY_TF32X3|VT_SGEMM_SKINNY_MMA_SYNC|VT_SGEMM_TILE32|VT_SGEMM_PANEL_TF32X3|VT_SGEMM_TALL_TF32X3|VT_SGEMM_PIPE128|VT_SGEMM_PIPE64|VT_SGEMM_PIPE64X128", "VT_HOST|VT_DEVICE|VT_HOST_AC_DEVICE_B"):
        for name in group.split("|"):
            m = re.search(r"\b%s\s*=\s*(\d+)" % name, text)
            assert m and int(m.group(1)) == getattr(native, name), name


def test_domain_errors_need_no_device(native):
    """Argument checks mirror validate_plan (reference backend.py:121-136) and come first."""
    import numpy as np

    a = np.zeros(64 * 64, dtype=np.int8)
    c = np.zeros(64 * 64, dtype=np.int32)
    cases = [((8, 16, 16), "m=8 must be >= dim=16"), ((16, 16, 33), "k=33 must be divisible by dim=16"),
             ((16, 24, 16), "n=24 must be divisible by dim=16"), ((16, 16, 131072), "overflow bound violated")]
    for (m, n, k), text in cases:
        with pytest.raises(native.NativeError) as info:
            native.i8gemm(a, a, c, m, n, k)
        assert info.value.code == native.VT_ERR_INVALID and text in info.value.message
    with pytest.raises(native.NativeError) as info:
        native.i8gemm(0, a, c, 16, 16, 16)
    assert info.value.code == native.VT_ERR_INVALID
    with pytest.raises(native.NativeError) as info:
        native.i8gemm(a, a, c, 16, 16, 16, raster=9)
    assert info.value.code == native.VT_ERR_INVALID
    with pytest.raises(native.NativeError) as info:
        native.i8gemm_shared_b(a, a, c, 2, 16, 16, 16, acc_rows=24)
    assert "accumulator_rows" in info.value.message
    f = np.zeros(16, dtype=np.float32)
    with pytest.raises(native.NativeError):
        native.sgemm(f, f, f, 0, 4, 4)
    with pytest.raises(native.NativeError):
        native.sgemm(f, f, f, 4, 4, 4, variant=17)
    off = np.array([0], dtype=np.int64)
    with pytest.raises(native.NativeError) as info:   # an A tile reaching past the buffer
        native.i8_tile_program(a, 255, a, 256, c, 256, 16, 16, 16, off, np.array([0, 1], dtype=np.int64), off, off)
    assert info.value.code == native.VT_ERR_PROGRAM
    with pytest.raises(native.NativeError) as info:   # more products than int32 can hold
        native.i8_tile_program(a, 256, a, 256, c, 256, 16, 16, 16, off, np.array([0, 8192], dtype=np.int64),
                               np.zeros(8192, dtype=np.int64), np.zeros(8192, dtype=np.int64))
    assert info.value.code == native.VT_ERR_OVERFLOW
    assert native.launch_count() == 0


def test_missing_library_fails_loudly(native, monkeypatch, tmp_path):
    monkeypatch.setattr(native, "_lib", None)
    monkeypatch.setattr(native, "LIB_PATH", tmp_path / "absent.so")
    with pytest.raises(native.NativeError) as info:
        native.lib()
    assert "no CPU fallback" in str(info.value)
