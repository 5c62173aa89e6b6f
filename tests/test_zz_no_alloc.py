"""The allocation-free skinny fp32 entry point (vt_sgemm_skinny_static_scratch).

It serves embedders whose own memory pool already owns the GPU, so the library must not call
cudaMalloc on their behalf; its K-split scratch is a fixed array inside the library image.  The test
calls it through the C ABI twice in a row — different shapes, so the second call runs over the first
call's leftovers in the shared array — and checks each result against the existing vt_sgemm skinny
path within the suite's fp32 tolerance (relative Frobenius error <= 1e-5; the two paths run the same
kernels, so they are in fact bit-identical).  The file sorts last so that a run that stops at the
first failure has already run every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-5


def relfro(c, ref):
    return float((c.double() - ref.double()).norm() / ref.double().norm())


def test_static_scratch_matches_workspace_path_two_calls_in_a_row(native):
    import torch

    st = native.torch_stream()
    gen = torch.Generator(device="cuda").manual_seed(4242)
    cases = []
    for (m, n, k) in ((16, 8192, 8192), (7, 1024, 4096)):
        A = torch.rand((m, k), device="cuda", generator=gen) * 2 - 1
        B = torch.rand((k, n), device="cuda", generator=gen) * 2 - 1
        want = torch.full((m, n), float("nan"), device="cuda")
        native.sgemm(A, B, want, m, n, k, variant=native.VT_SGEMM_SKINNY, where=native.VT_DEVICE, stream=st)
        native.sync(0, st)
        cases.append((m, n, k, A, B, want, torch.full((m, n), float("nan"), device="cuda")))
    # The point of the entry point: it takes no device memory.  After one warm-up call (the first call on a
    # device looks up the array's address and loads the kernels), the free memory the driver reports must be
    # the same before and after the two calls; every tensor they use exists already.
    warm = torch.zeros((1, 64), device="cuda")
    native.sgemm_skinny_static_scratch(torch.zeros((1, 64), device="cuda"), torch.zeros((64, 64), device="cuda"), warm,
                                       1, 64, 64, stream=st)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for (m, n, k, A, B, want, got) in cases:
        native.sgemm_skinny_static_scratch(A, B, got, m, n, k, stream=st)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the allocation-free entry point changed the device's free memory"
    for (m, n, k, A, B, want, got) in cases:
        assert not torch.isnan(got).any()
        assert relfro(got, want) <= TOL
        assert torch.equal(got, want)
        ref = A.double() @ B.double()
        assert relfro(got, ref) <= TOL


def test_static_scratch_refuses_what_does_not_fit(native):
    """Sizes are checked before anything is touched, so small dummy buffers suffice here."""
    import torch

    dummy = torch.zeros(64, device="cuda")
    with pytest.raises(native.NativeError) as info:      # seven K splits of 16 x 64000 partials = 27 MiB > 8 MiB
        native.sgemm_skinny_static_scratch(dummy, dummy, dummy, 16, 64000, 8192, stream=native.torch_stream())
    assert info.value.code == native.VT_ERR_UNSUPPORTED
    assert "static array holds %d" % native.SKINNY_STATIC_SCRATCH_BYTES in info.value.message
    with pytest.raises(native.NativeError):              # not a skinny shape
        native.sgemm_skinny_static_scratch(dummy, dummy, dummy, 17, 64, 64)
    with pytest.raises(native.NativeError):
        native.sgemm_skinny_static_scratch(0, dummy, dummy, 16, 64, 64)
