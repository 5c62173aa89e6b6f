"""Parity of the CUDA fp32 path: relative Frobenius error <= 1e-5 against float64 (the stated
tolerance), agreement with the generated-OpenMP-C restatement on the same seeded inputs, and the
drop-in `benchmark_matmul` entry point."""
import numpy as np
import pytest

import loopnest_oracle as lo

pytestmark = pytest.mark.gpu

TOL = 1e-5   # relative Frobenius error against a float64 product


def relfro(c, ref):
    return float(np.linalg.norm(c.astype(np.float64) - ref) / np.linalg.norm(ref))


def uniform(rng, shape):
    return (rng.random(shape, dtype=np.float32) * 2 - 1)


@pytest.mark.parametrize("variant", [0, 1, 2, 4, 7, 10, 11, 12])
def test_shapes_against_float64(native, variant):
    rng = np.random.default_rng(20260917 + 1)
    for (m, n, k) in ((256, 256, 256), (1, 1, 1), (5, 3, 2), (77, 130, 33), (300, 200, 100), (128, 128, 16),
                      (129, 127, 17), (512, 384, 1000), (1024, 1024, 1024), (64, 2048, 96), (40, 36, 260), (512, 512, 512),
                      (33, 4, 4)):
        if variant in (4, 7, 10, 11, 12) and (n % 4 or k % 4):
            with pytest.raises(native.NativeError):     # the tensor-core variant needs 16-byte row pitches
                native.sgemm(uniform(rng, (m, k)), uniform(rng, (k, n)), np.zeros((m, n), np.float32), m, n, k,
                             variant=variant)
            continue
        a, b = uniform(rng, (m, k)), uniform(rng, (k, n))
        c = np.full((m, n), np.nan, dtype=np.float32)
        native.sgemm(a, b, c, m, n, k, variant=variant)
        assert relfro(c, a.astype(np.float64) @ b.astype(np.float64)) <= TOL, (m, n, k)


@pytest.mark.parametrize("variant", [10, 12, 11, 7])
def test_k_split_every_count_and_bit_identical_repeats(native, variant):
    """The FFMA kernels that split K over several CTAs per output tile (the pipelined kernel over the CTAs of a
    cluster, through their shared memory; the 32-wide kernel through scratch memory and a ticket per tile): every
    split count the hook can force, on shapes with ragged edges, K not a multiple of a stage, more splits than K
    has stages and more tiles than one wave of clusters holds, against float64; and the same call twice gives the
    same bits, because partial tiles are added in split order whichever CTA finishes last."""
    import torch
    st = native.torch_stream()
    gen = torch.Generator(device="cuda").manual_seed(811)
    shapes = ((640, 640, 640), (200, 300, 400), (77, 132, 36), (128, 128, 4096), (1, 4, 64), (384, 520, 1000),
              (1500, 1400, 260), (64, 64, 8192))
    try:
        for (m, n, k) in shapes:
            A = torch.rand((m, k), device="cuda", generator=gen) * 2 - 1
            B = torch.rand((k, n), device="cuda", generator=gen) * 2 - 1
            ref = (A.double() @ B.double()).cpu().numpy()
            for splits in ((0, 1, 2, 3, 5, 8) if variant != 7 else (0, 1, 2, 4, 7, 16)):
                native.test_set_sgemm_splits(splits)
                out = []
                for rep in range(2):
                    C = torch.full((m, n), float("nan"), device="cuda")
                    native.sgemm(A, B, C, m, n, k, variant=variant, where=native.VT_DEVICE, stream=st)
                    native.sync(0, st)
                    out.append(C)
                assert relfro(out[0].cpu().numpy(), ref) <= TOL, (m, n, k, splits)
                assert torch.equal(out[0], out[1]), (m, n, k, splits)
    finally:
        native.test_set_sgemm_splits(0)


def test_tf32x3_error_does_not_grow_with_k(native):
    """The 3xTF32 variant folds at most 128 values of K into one tensor-core accumulator; its error
    must stay far inside the tolerance for long reductions and for same-sign data (the worst case for
    a truncating accumulator)."""
    import torch
    gen = torch.Generator(device="cuda").manual_seed(7)
    st = native.torch_stream()
    for (m, n, k) in ((512, 512, 16384), (1024, 768, 4096), (260, 516, 1028)):
        for positive in (False, True):
            A = torch.rand((m, k), device="cuda", generator=gen)
            B = torch.rand((k, n), device="cuda", generator=gen)
            if not positive:
                A, B = A * 2 - 1, B * 2 - 1
            C = torch.full((m, n), float("nan"), device="cuda")
            native.sgemm(A, B, C, m, n, k, variant=native.VT_SGEMM_TF32X3, where=native.VT_DEVICE, stream=st)
            native.sync(0, st)
            ref = A.double() @ B.double()
            assert float((C.double() - ref).norm() / ref.norm()) <= TOL / 4, (m, n, k, positive)


def test_256_cubed_vs_generated_c(native, liboracle):
    """The 256^3 demo workload: uniform[-1,1) fp32 256^3, C zero-initialised; the generated OpenMP nests
    (float64, as the reference emits them) are the float64 reference."""
    rng = np.random.default_rng(20260917 + 1)
    m = n = k = 256
    a, b = uniform(rng, (m, k)), uniform(rng, (k, n))
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    ref_tuned, ref_naive = np.zeros((m, n)), np.zeros((m, n))
    liboracle.oracle_dgemm_tuned(a64.ctypes.data, b64.ctypes.data, ref_tuned.ctypes.data, m, n, k)
    liboracle.oracle_dgemm_naive(a64.ctypes.data, b64.ctypes.data, ref_naive.ctypes.data, m, n, k)
    assert relfro(ref_tuned, ref_naive) < 1e-14
    for variant in (0, 1, 2, 4, 7):
        c = np.zeros((m, n), dtype=np.float32)
        native.sgemm(a, b, c, m, n, k, variant=variant)
        assert relfro(c, ref_tuned) <= TOL and relfro(c, a64 @ b64) <= TOL


@pytest.mark.parametrize("variant", [3, 5, 6])
def test_skinny_kernel(native, variant):
    """Variant 5 runs tcgen05 where K % 4 == 0 and the mma.sync form elsewhere; the shapes cover one CTA
    per slab, whole K ranges per CTA, left-over CTAs that run through several slabs, more slabs than
    CTAs, ragged N and K, and the K-split tickets returning to zero between calls."""
    rng = np.random.default_rng(20260917 + 5)
    for (m, n, k) in ((16, 8192, 8192), (16, 1024, 640), (7, 1024, 640), (1, 512, 4096), (16, 516, 100),
                      (3, 128, 64), (16, 132, 31), (5, 4, 7), (9, 260, 8), (16, 16384, 4096), (12, 60000, 512),
                      (16, 4096, 16384), (2, 2048, 2050), (16, 22700, 4001), (15, 20040, 3995)):
        a, b = uniform(rng, (m, k)), uniform(rng, (k, n))
        c = np.full((m, n), np.nan, dtype=np.float32)
        native.sgemm(a, b, c, m, n, k, variant=variant)
        assert relfro(c, a.astype(np.float64) @ b.astype(np.float64)) <= TOL, (m, n, k)
        c2 = np.full((m, n), np.nan, dtype=np.float32)
        native.sgemm(a, b, c2, m, n, k, variant=variant)
        assert np.array_equal(c, c2)      # fixed summation order: bit-reproducible
    with pytest.raises(native.NativeError):
        native.sgemm(uniform(rng, (17, 64)), uniform(rng, (64, 64)), np.zeros((17, 64), np.float32), 17, 64, 64,
                     variant=variant)


def test_row_panel_kernel(native):
    """PANEL_TF32X3: panels of 16, 32, 64 and 128 rows of A, one launch per 128 rows; ragged N and K, a last
    panel of a few rows, K splits, same-sign data (the worst case for a truncating accumulator), reruns
    bit-identical, and the automatic choice for few rows against a large B."""
    import torch
    gen = torch.Generator(device="cuda").manual_seed(20260917 + 8)
    st = native.torch_stream()
    for (m, n, k) in ((17, 512, 512), (32, 1024, 1024), (33, 1024, 1028), (48, 1000, 996), (64, 2048, 1024),
                      (65, 1284, 2052), (100, 4096, 512), (128, 1024, 4096), (129, 1024, 1024), (200, 2052, 1000),
                      (256, 4096, 4096), (300, 1024, 1024), (7, 1028, 1000), (128, 8192, 8192), (40, 16384, 2048),
                      (96, 132, 8192), (20, 4, 4), (128, 60000, 256)):
        for positive in (False, True):
            A = torch.rand((m, k), device="cuda", generator=gen)
            B = torch.rand((k, n), device="cuda", generator=gen)
            if not positive:
                A, B = A * 2 - 1, B * 2 - 1
            ref = A.double() @ B.double()
            C = torch.full((m, n), float("nan"), device="cuda")
            native.sgemm(A, B, C, m, n, k, variant=native.VT_SGEMM_PANEL_TF32X3, where=native.VT_DEVICE, stream=st)
            native.sync(0, st)
            assert float((C.double() - ref).norm() / ref.norm()) <= TOL / 3, (m, n, k, positive)
            C2 = torch.full((m, n), float("nan"), device="cuda")
            native.sgemm(A, B, C2, m, n, k, variant=native.VT_SGEMM_PANEL_TF32X3, where=native.VT_DEVICE, stream=st)
            native.sync(0, st)
            assert torch.equal(C, C2), (m, n, k)
    A = torch.rand((96, 4096), device="cuda", generator=gen) * 2 - 1
    B = torch.rand((4096, 4096), device="cuda", generator=gen) * 2 - 1
    C, Cp = torch.empty((96, 4096), device="cuda"), torch.empty((96, 4096), device="cuda")
    native.sgemm(A, B, C, 96, 4096, 4096, where=native.VT_DEVICE, stream=st)
    native.sgemm(A, B, Cp, 96, 4096, 4096, variant=native.VT_SGEMM_PANEL_TF32X3, where=native.VT_DEVICE, stream=st)
    native.sync(0, st)
    assert torch.equal(C, Cp)              # the automatic choice for this shape is the panel kernel
    with pytest.raises(native.NativeError):
        native.sgemm(torch.zeros((32, 66), device="cuda"), torch.zeros((66, 64), device="cuda"),
                     torch.zeros((32, 64), device="cuda"), 32, 64, 66, variant=native.VT_SGEMM_PANEL_TF32X3,
                     where=native.VT_DEVICE, stream=st)


def test_tall_kernel(native):
    """TALL_TF32X3: A streamed in slabs of 128 rows against panels of up to 16, 32, 64 or 128 columns (wider C in
    several panels); ragged M, N and K, K splits, one slab, same-sign data, reruns bit-identical, the automatic
    choice, and refusal of N % 4 != 0 or K % 4 != 0."""
    import torch
    gen = torch.Generator(device="cuda").manual_seed(20260917 + 10)
    st = native.torch_stream()
    for (m, n, k) in ((128, 16, 128), (128, 4, 64), (300, 12, 100), (1000, 32, 1028), (999, 64, 516), (2048, 8, 2048),
                      (4096, 48, 512), (130, 20, 36), (1, 4, 4), (8192, 16, 8192), (8192, 64, 8192), (65536, 16, 1024),
                      (1024, 64, 16384), (20000, 36, 260), (257, 64, 8192), (100, 16, 65536), (512, 128, 512),
                      (1000, 200, 1000), (700, 256, 2048), (300, 132, 260), (4096, 300, 1024), (8192, 128, 8192)):
        for positive in (False, True):
            A = torch.rand((m, k), device="cuda", generator=gen)
            B = torch.rand((k, n), device="cuda", generator=gen)
            if not positive:
                A, B = A * 2 - 1, B * 2 - 1
            ref = A.double() @ B.double()
            C = torch.full((m, n), float("nan"), device="cuda")
            native.sgemm(A, B, C, m, n, k, variant=native.VT_SGEMM_TALL_TF32X3, where=native.VT_DEVICE, stream=st)
            native.sync(0, st)
            assert float((C.double() - ref).norm() / ref.norm()) <= TOL / 3, (m, n, k, positive)
            C2 = torch.full((m, n), float("nan"), device="cuda")
            native.sgemm(A, B, C2, m, n, k, variant=native.VT_SGEMM_TALL_TF32X3, where=native.VT_DEVICE, stream=st)
            native.sync(0, st)
            assert torch.equal(C, C2), (m, n, k)
    A = torch.rand((4096, 4096), device="cuda", generator=gen) * 2 - 1
    B = torch.rand((4096, 32), device="cuda", generator=gen) * 2 - 1
    C, Ct = torch.empty((4096, 32), device="cuda"), torch.empty((4096, 32), device="cuda")
    native.sgemm(A, B, C, 4096, 32, 4096, where=native.VT_DEVICE, stream=st)
    native.sgemm(A, B, Ct, 4096, 32, 4096, variant=native.VT_SGEMM_TALL_TF32X3, where=native.VT_DEVICE, stream=st)
    native.sync(0, st)
    assert torch.equal(C, Ct)              # the automatic choice for this shape is the tall kernel
    for (m, n, k) in ((256, 18, 256), (256, 16, 258)):
        with pytest.raises(native.NativeError):
            native.sgemm(torch.zeros((m, k), device="cuda"), torch.zeros((k, n), device="cuda"),
                         torch.zeros((m, n), device="cuda"), m, n, k, variant=native.VT_SGEMM_TALL_TF32X3,
                         where=native.VT_DEVICE, stream=st)


def test_non_finite_inputs(native):
    """Infinities and NaNs: the true-fp32 kernels give IEEE results (same NaN and infinity pattern as a float32
    product).  The 3xTF32 kernels compute x * inf as hi * inf + lo * inf, which is NaN where lo is zero or of the
    other sign, so there only the rows and columns that hold a non-finite input may differ, and only by NaN
    standing where the float32 product has an infinity; everything else stays inside the tolerance."""
    import torch
    gen = torch.Generator(device="cuda").manual_seed(20260917 + 9)
    st = native.torch_stream()
    for (m, n, k, variants) in ((16, 1024, 1024, (3, 5, 6)), (96, 2048, 2048, (2, 8)), (512, 1024, 1024, (1, 2, 4, 7)),
                                (2048, 32, 1024, (7, 9)), (64, 64, 64, (0,))):
        A = torch.rand((m, k), device="cuda", generator=gen) * 2 - 1
        B = torch.rand((k, n), device="cuda", generator=gen) * 2 - 1
        A[0, 0], B[3, 5], A[2, 2] = float("inf"), float("-inf"), float("nan")
        ref = (A.double() @ B.double()).float()
        touched = torch.zeros((m, n), dtype=torch.bool, device="cuda")
        touched[0, :] = True
        touched[2, :] = True
        touched[:, 5] = True
        for variant in variants:
            C = torch.empty((m, n), device="cuda")
            native.sgemm(A, B, C, m, n, k, variant=variant, where=native.VT_DEVICE, stream=st)
            native.sync(0, st)
            clean = ~touched
            err = float((C[clean].double() - ref[clean].double()).norm() / ref[clean].double().norm())
            assert err <= TOL, (m, n, k, variant)
            assert bool(torch.isnan(C[2]).all()), (m, n, k, variant)
            if variant in (1, 2, 3, 7) or (variant == 0 and m == 64):
                assert torch.equal(torch.isnan(C), torch.isnan(ref)), (m, n, k, variant)
                assert torch.equal(C[torch.isinf(ref)], ref[torch.isinf(ref)]), (m, n, k, variant)
            else:
                assert bool((torch.isnan(C) | (C == ref))[torch.isinf(ref)].all()), (m, n, k, variant)


def test_8192_cubed_and_skinny_fp32(native):
    """The large fp32 workloads: 8192^3 (device resident, checked on sampled rows in float64 on the GPU)
    and the skinny 16 x 8192 x 8192 shape."""
    import torch
    M = N = K = 8192
    gen = torch.Generator(device="cuda").manual_seed(20260917 + 5)
    A = torch.rand((M, K), device="cuda", generator=gen) * 2 - 1
    B = torch.rand((K, N), device="cuda", generator=gen) * 2 - 1
    C = torch.full((M, N), float("nan"), device="cuda")
    st = native.torch_stream()
    rows = torch.arange(0, M, 64, device="cuda")
    ref = A[rows].double() @ B.double()
    for variant in (native.VT_SGEMM_AUTO, native.VT_SGEMM_TILE128, native.VT_SGEMM_TF32X3):
        C.fill_(float("nan"))
        native.sgemm(A, B, C, M, N, K, variant=variant, where=native.VT_DEVICE, stream=st)
        native.sync(0, st)
        assert float((C[rows].double() - ref).norm() / ref.norm()) <= TOL
        assert not torch.isnan(C).any()
    C16 = torch.full((16, N), float("nan"), device="cuda")
    native.sgemm(A[:16], B, C16, 16, N, K, where=native.VT_DEVICE, stream=st)
    native.sync(0, st)
    ref16 = A[:16].double() @ B.double()
    assert float((C16.double() - ref16).norm() / ref16.norm()) <= TOL


def test_benchmark_matmul_drop_in(native, golden_cpu_gemm):
    """The reference's entry point on its own operand pattern: same keys, same four cells."""
    from veritac_b200.CodeGen import runner
    for run in golden_cpu_gemm["benchmark_matmul"]:
        M, K, N = run["M"], run["K"], run["N"]
        stmt = lo.matmul_stmt(M, K, N)
        if run["schedule"]:
            stmt = lo.apply_tactics(stmt, lo.README_SCHEDULE)
        r = runner.benchmark_matmul(stmt, M, K, N, num_runs=3)
        assert {"c_time_ms", "numpy_time_ms", "speedup", "correct", "c_first_values", "np_first_values"} <= set(r)
        assert r["correct"] is True
        assert r["c_first_values"] == run["c_first_values"] and r["np_first_values"] == run["np_first_values"]
        assert r["rel_frobenius_error"] == 0.0      # small-integer operands: fp32 is exact
        assert r["c_time_ms"] > 0 and r["speedup"] > 0


def test_demos_run_end_to_end(native, capsys):
    """The demo callers on this back end: the reference's gemm_demo flow, and the Gemmini demo that puts measured
    GPU time beside the modeled traffic."""
    from veritac_b200.examples import gemm_demo, gemmini_gemm_demo
    assert gemm_demo.main(["--dim", "256", "--runs", "2"]) == 0
    assert "correct: True" in capsys.readouterr().out
    report = gemmini_gemm_demo.run_demo(64, 64, 64, repeats=3)
    assert report["verified"] and report["winner"]["schedule"] == "reuse_b"
    assert report["mismatches"] == {} and report["controls_bit_exact"] is True
    assert [s["accepted"] for s in report["search"]] == [True, True]
    names = [r["stream"] for r in report["rows"]]
    assert names[0] == "baseline" and names[-1] == "winner(reuse_b)" and all(r["gpu_time_ms"] > 0 for r in report["rows"])
    # the model ranks the winner's traffic below the baseline's; the report shows both beside the measured time
    assert report["rows"][-1]["modeled_input_bytes"] <= report["rows"][0]["modeled_input_bytes"]
    assert gemmini_gemm_demo.main(["--m", "32", "--n", "16", "--k", "16", "--repeats", "2"]) == 0
    assert "winner by modeled objective" in capsys.readouterr().out
    from veritac_b200.examples import llm_gemm_demo
    assert llm_gemm_demo.main(["--mock", "--dim", "256", "--runs", "2"]) == 0
    out = capsys.readouterr().out
    assert out.count("verifier: applied") == 5 and "correct: True" in out
    assert "kernel the library chose for 256x256x256: TILE32" in out and "tiles point at: TILE32" in out


def test_stream_order_holds_across_overlapped_launches(native):
    """Back-to-back calls where each product reads what the one before it wrote (X <- X . B through two
    buffers; skinny, panel, small and 3xTF32 kernels) must give the bits of the same chain run with a synchronisation after
    every call: these kernels start their set-up before the previous kernel on the stream has finished and may
    touch memory only after it has."""
    import torch
    st = native.torch_stream()
    gen = torch.Generator(device="cuda").manual_seed(77)
    for (m, n) in ((16, 2048), (8, 4096), (96, 2048), (256, 256), (1024, 1024)):
        B = (torch.rand((n, n), device="cuda", generator=gen) * 2 - 1) / (n ** 0.5) * 1.7
        X0 = torch.rand((m, n), device="cuda", generator=gen) * 2 - 1
        results = []
        for synced in (True, False):
            bufs = [X0.clone(), torch.zeros_like(X0)]
            for step in range(12):
                src, dst = bufs[step & 1], bufs[1 - (step & 1)]
                native.sgemm(src, B, dst, m, n, n, where=native.VT_DEVICE, stream=st)
                if synced:
                    native.sync(0, st)
            native.sync(0, st)
            results.append(bufs[0].clone())
        assert torch.isfinite(results[0]).all() and float(results[0].abs().max()) > 0
        assert torch.equal(results[0], results[1]), (m, n)


@pytest.mark.parametrize("variant,shape", [(1, (512, 384, 640)), (2, (320, 448, 200)), (9, (16384, 32, 512)),
                                           (8, (96, 1024, 1024)), (4, (512, 512, 512)), (10, (640, 640, 640)),
                                           (12, (768, 768, 768)), (7, (256, 256, 4096))])
def test_inputs_written_by_the_kernel_before(native, variant, shape):
    """B is rewritten and C poisoned by ordinary kernels right before each product, with no synchronisation:
    a product that started reading or writing before those kernels had finished would see the other B or lose
    its output to the poison."""
    import torch
    m, n, k = shape
    st = native.torch_stream()
    gen = torch.Generator(device="cuda").manual_seed(78)
    A = torch.rand((m, k), device="cuda", generator=gen) * 2 - 1
    Bs = [torch.rand((k, n), device="cuda", generator=gen) * 2 - 1 for _ in range(2)]
    Bw = torch.empty_like(Bs[0])
    C = torch.empty((m, n), device="cuda")
    for rep in range(7):
        Bw.copy_(Bs[rep & 1])
        C.fill_(float("nan"))
        native.sgemm(A, Bw, C, m, n, k, variant=variant, where=native.VT_DEVICE, stream=st)
    native.sync(0, st)
    ref = (A.double() @ Bs[0].double()).cpu().numpy()
    assert relfro(C.cpu().numpy(), ref) <= TOL


def test_automatic_choice_at_its_boundaries(native):
    """vt_sgemm_auto_variant: what VT_SGEMM_AUTO launches, asked without launching.  The streaming tensor-core
    kernels keep one arrival counter per 128-wide slab (4096 of them); shapes with more slabs must fall through to
    kernels that can serve them instead of being refused."""
    nv = native
    assert nv.sgemm_auto_variant(16, 8192, 8192) == nv.VT_SGEMM_SKINNY_TF32X3
    assert nv.sgemm_auto_variant(64, 8192, 8192) == nv.VT_SGEMM_PANEL_TF32X3
    assert nv.sgemm_auto_variant(8192, 16, 8192) == nv.VT_SGEMM_TALL_TF32X3
    assert nv.sgemm_auto_variant(8192, 8192, 8192) == nv.VT_SGEMM_TF32X3
    assert nv.sgemm_auto_variant(256, 256, 256) == nv.VT_SGEMM_TILE32
    # mid-sized products go to the pipelined FFMA kernel with its cluster K split, long-K small ones to the 32-wide
    # kernel with its own split, cubes from ~900 up to the tensor cores
    assert nv.sgemm_auto_variant(640, 640, 640) in (nv.VT_SGEMM_PIPE128, nv.VT_SGEMM_PIPE64X128, nv.VT_SGEMM_PIPE64)
    assert nv.sgemm_auto_variant(512, 512, 8192) in (nv.VT_SGEMM_PIPE128, nv.VT_SGEMM_PIPE64X128, nv.VT_SGEMM_PIPE64)
    assert nv.sgemm_auto_variant(256, 256, 8192) == nv.VT_SGEMM_TILE32
    assert nv.sgemm_auto_variant(128, 128, 65536) == nv.VT_SGEMM_TILE32
    assert nv.sgemm_auto_variant(1024, 1024, 1024) == nv.VT_SGEMM_TF32X3
    limit = 4096 * 128
    assert nv.sgemm_auto_variant(16, limit, 1024) == nv.VT_SGEMM_SKINNY_TF32X3
    assert nv.sgemm_auto_variant(16, limit + 128, 1024) not in (nv.VT_SGEMM_SKINNY_TF32X3, nv.VT_SGEMM_PANEL_TF32X3)
    assert nv.sgemm_auto_variant(64, limit + 128, 1024) != nv.VT_SGEMM_PANEL_TF32X3
    assert nv.sgemm_auto_variant(limit, 16, 1024) == nv.VT_SGEMM_TALL_TF32X3
    assert nv.sgemm_auto_variant(limit + 128, 16, 1024) != nv.VT_SGEMM_TALL_TF32X3
    with pytest.raises(nv.NativeError):
        nv.sgemm_auto_variant(0, 16, 16)

def test_device_calls_capture_into_a_cuda_graph(native):
    """Device-pointer calls only enqueue work, so after one eager pass (which sizes the workspace and sets the
    kernels' attributes) a sequence of them can be captured into a CUDA graph and replayed: the int8 pair kernel and
    every fp32 family (32-wide with and without its K split, the pipelined kernel with its cluster split, the
    streaming kernels for few rows and few columns, 3xTF32 with its lo-part pass), launched with programmatic
    stream serialization and, for the split, as clusters.  Every replay must give the bits of the eager pass."""
    import torch
    gen = torch.Generator(device="cuda").manual_seed(9)
    A8 = torch.randint(-128, 128, (1024, 2048), dtype=torch.int8, device="cuda", generator=gen)
    B8 = torch.randint(-128, 128, (2048, 1536), dtype=torch.int8, device="cuda", generator=gen)
    C8 = torch.zeros((1024, 1536), dtype=torch.int32, device="cuda")
    cases = []
    for (m, n, k) in ((256, 256, 256), (640, 640, 640), (16, 4096, 4096), (256, 256, 4096), (1024, 1024, 1024),
                      (96, 2048, 2048), (2048, 16, 2048)):
        cases.append((m, n, k, torch.rand((m, k), device="cuda", generator=gen) * 2 - 1,
                      torch.rand((k, n), device="cuda", generator=gen) * 2 - 1, torch.zeros((m, n), device="cuda")))

    def enqueue(handle):
        native.i8gemm(A8, B8, C8, 1024, 1536, 2048, where=native.VT_DEVICE, stream=handle)
        for (m, n, k, A, B, C) in cases:
            native.sgemm(A, B, C, m, n, k, where=native.VT_DEVICE, stream=handle)

    s = torch.cuda.Stream()
    handle = int(s.cuda_stream)
    with torch.cuda.stream(s):
        enqueue(handle)
    s.synchronize()
    native.sync(0, handle)
    want8, want = C8.clone(), [c[5].clone() for c in cases]
    assert torch.equal(want8, (A8.double() @ B8.double()).to(torch.int32))
    for (m, n, k, A, B, C) in cases:
        assert relfro(C.cpu().numpy(), (A.double() @ B.double()).cpu().numpy()) <= TOL
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s):
        enqueue(handle)
    for rep in range(3):
        C8.fill_(-1)
        for c in cases:
            c[5].fill_(float("nan"))
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(C8, want8), rep
        for c, w in zip(cases, want):
            assert torch.equal(c[5], w), (c[:3], rep)
    native.sync(0, handle)
