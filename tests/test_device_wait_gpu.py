"""Failure detection on the device: every wait in the kernels is bounded, and a wait that runs out ends the
kernel with a status word instead of a hang (the fail-closed idiom of the reference's interpreter,
specializations/gemmini_gemm/backend.py:164-196, carried to the device).

Nothing here traps, faults or spins without a limit.  The failures are made by the host: a barrier that
nothing completes, and an operand producer told to stop early, so that the waits on it run out after about a
millisecond.  The kernels then tear their pipelines down and return; vt_sync reports VT_ERR_DEVICE_WAIT, the
status word, tickets and flags are cleared, and the next ordinary call on the same device is exact."""
import numpy as np
import pytest

import gemmini_oracle as go

pytestmark = pytest.mark.gpu

SHORT = 4_000_000        # cycles: about 2 ms


def exact_call(native, m, n, k, seed, variant=3):
    import torch
    gen = torch.Generator(device="cuda").manual_seed(seed)
    A = torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda", generator=gen)
    B = torch.randint(-128, 128, (k, n), dtype=torch.int8, device="cuda", generator=gen)
    C = torch.full((m, n), -2**31, dtype=torch.int32, device="cuda")
    st = native.torch_stream()
    native.i8gemm(A, B, C, m, n, k, variant=variant, where=native.VT_DEVICE, stream=st)
    native.sync(0, st)
    assert torch.equal(C, (A.double() @ B.double()).to(torch.int32)), (m, n, k)


def test_a_wait_that_runs_out_is_reported_and_cleared(native):
    st = native.torch_stream()
    native.sync(0, st)
    try:
        native.test_set_wait_hooks(0, SHORT, -1)
        native.test_expire_wait(0, st)
        with pytest.raises(native.NativeError) as err:
            native.sync(0, st)
        assert err.value.code == native.VT_ERR_DEVICE_WAIT
        assert "status 102" in err.value.message
    finally:
        native.test_set_wait_hooks(0, 0, -1)
    native.sync(0, st)                      # the status word was cleared by the failing check
    exact_call(native, 384, 512, 640, 1)


@pytest.mark.parametrize("shape", [(512, 512, 4096), (1024, 8192, 8192)])
def test_pair_kernel_tears_down_when_its_peer_stops(native, shape):
    """The odd CTA of every pair stops feeding operands at the sixth ring fill.  The even CTA's wait for that
    fill runs out, both CTAs agree to give up, the even CTA settles the books of its barriers and waits for
    the copies in flight, and the kernel returns.  The second shape gives most pairs two tiles, so the give-up
    comes with accumulators in both states."""
    import torch
    m, n, k = shape
    st = native.torch_stream()
    gen = torch.Generator(device="cuda").manual_seed(7)
    A = torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda", generator=gen)
    B = torch.randint(-128, 128, (k, n), dtype=torch.int8, device="cuda", generator=gen)
    C = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    try:
        native.test_set_wait_hooks(0, SHORT, 5)
        native.i8gemm(A, B, C, m, n, k, variant=native.VT_I8_CTA_PAIR, where=native.VT_DEVICE, stream=st)
        with pytest.raises(native.NativeError) as err:
            native.sync(0, st)
        assert err.value.code == native.VT_ERR_DEVICE_WAIT
    finally:
        native.test_set_wait_hooks(0, 0, -1)
    native.sync(0, st)
    for rep in range(2):
        exact_call(native, m, n, k, 11 + rep)
