"""Seeded random shapes through every kernel variant (device-resident operands, C poisoned): the sweep that
found the one synchronisation fault of this code base, kept as a regression test.  int8 against the exact
product, fp32 against float64 within the 1e-5 relative Frobenius contract."""
import numpy as np
import pytest

import gemmini_oracle as go

pytestmark = pytest.mark.gpu
TOL = 1e-5


def relfro(c, ref):
    return float(np.linalg.norm(c.astype(np.float64) - ref) / np.linalg.norm(ref))


def test_random_skinny_shapes(native):
    import torch
    rng = np.random.default_rng(20260917 + 21)
    st = native.torch_stream()
    for _ in range(48):
        m = int(rng.integers(1, 17))
        n = 4 * int(rng.integers(1, 8000))
        k = int(rng.integers(1, 4200))
        if rng.random() < 0.5:
            k = 4 * (k // 4 + 1)
        a = rng.random((m, k), dtype=np.float32) * 2 - 1
        b = rng.random((k, n), dtype=np.float32) * 2 - 1
        ref = a.astype(np.float64) @ b.astype(np.float64)
        A, B = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        for variant in (3, 5, 6):
            for _rep in range(2):                      # the fault showed only now and then
                C = torch.full((m, n), float("nan"), device="cuda")
                native.sgemm(A, B, C, m, n, k, variant=variant, where=native.VT_DEVICE, stream=st)
                native.sync(0, st)
                assert relfro(C.cpu().numpy(), ref) <= TOL, (m, n, k, variant)


def test_random_fp32_shapes(native):
    import torch
    rng = np.random.default_rng(20260917 + 22)
    st = native.torch_stream()
    for _ in range(24):
        m, n, k = (int(x) for x in rng.integers(1, 1300, 3))
        if rng.random() < 0.6:
            n, k = 4 * (n // 4 + 1), 4 * (k // 4 + 1)
        a = rng.random((m, k), dtype=np.float32) * 2 - 1
        b = rng.random((k, n), dtype=np.float32) * 2 - 1
        ref = a.astype(np.float64) @ b.astype(np.float64)
        A, B = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        for variant in (0, 1, 2, 4, 7, 10, 11, 12):
            if variant in (4, 7, 10, 11, 12) and (n % 4 or k % 4):
                continue
            C = torch.full((m, n), float("nan"), device="cuda")
            native.sgemm(A, B, C, m, n, k, variant=variant, where=native.VT_DEVICE, stream=st)
            native.sync(0, st)
            assert relfro(C.cpu().numpy(), ref) <= TOL, (m, n, k, variant)


def test_random_row_panel_shapes(native):
    import torch
    rng = np.random.default_rng(20260917 + 24)
    st = native.torch_stream()
    for _ in range(40):
        m = int(rng.integers(1, 300))
        n = 4 * int(rng.integers(1, 3000))
        k = 4 * int(rng.integers(1, 1500))
        a = rng.random((m, k), dtype=np.float32) * 2 - 1
        b = rng.random((k, n), dtype=np.float32) * 2 - 1
        ref = a.astype(np.float64) @ b.astype(np.float64)
        A, B = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        for _rep in range(2):
            C = torch.full((m, n), float("nan"), device="cuda")
            native.sgemm(A, B, C, m, n, k, variant=native.VT_SGEMM_PANEL_TF32X3, where=native.VT_DEVICE, stream=st)
            native.sync(0, st)
            assert relfro(C.cpu().numpy(), ref) <= TOL, (m, n, k)


def test_random_tall_shapes(native):
    import torch
    rng = np.random.default_rng(20260917 + 25)
    st = native.torch_stream()
    for _ in range(40):
        m = int(rng.integers(1, 6000))
        n = 4 * int(rng.integers(1, 17 if rng.random() < 0.6 else 80))
        k = 4 * int(rng.integers(1, 1500))
        a = rng.random((m, k), dtype=np.float32) * 2 - 1
        b = rng.random((k, n), dtype=np.float32) * 2 - 1
        ref = a.astype(np.float64) @ b.astype(np.float64)
        A, B = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        for _rep in range(2):
            C = torch.full((m, n), float("nan"), device="cuda")
            native.sgemm(A, B, C, m, n, k, variant=native.VT_SGEMM_TALL_TF32X3, where=native.VT_DEVICE, stream=st)
            native.sync(0, st)
            assert relfro(C.cpu().numpy(), ref) <= TOL, (m, n, k)


def test_random_int8_shapes(native):
    import torch
    rng = np.random.default_rng(20260917 + 23)
    st = native.torch_stream()
    for _ in range(24):
        m, n, k = (16 * int(x) for x in rng.integers(1, 100, 3))
        a = rng.integers(-128, 128, (m, k), dtype=np.int8)
        b = rng.integers(-128, 128, (k, n), dtype=np.int8)
        want = go.matmul_exact(a.reshape(-1), b.reshape(-1), m, n, k).reshape(m, n)
        A, B = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        for variant in (0, 1, 3, 4):
            C = torch.full((m, n), -2**31, dtype=torch.int32, device="cuda")
            native.i8gemm(A, B, C, m, n, k, variant=variant, raster=int(rng.integers(0, 4)),
                          batch_rows=int(rng.integers(1, 65)), where=native.VT_DEVICE, stream=st)
            native.sync(0, st)
            assert np.array_equal(C.cpu().numpy(), want), (m, n, k, variant)
