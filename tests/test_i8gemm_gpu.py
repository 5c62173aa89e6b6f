"""Parity of the CUDA int8 path with the oracle and with the reference's recorded results.
Everything goes through the C ABI (ctypes) or the drop-in Python entry points above it."""
import hashlib
import json

import numpy as np
import pytest

import gemmini_oracle as go
from conftest import commands_from_dicts

pytestmark = pytest.mark.gpu


def sha(obj):
    return hashlib.sha256(json.dumps(obj).encode()).hexdigest()


@pytest.fixture(scope="module")
def g(native):
    from veritac_b200.CodeGen import gemmini
    return gemmini


@pytest.fixture(scope="module")
def lowering(native):
    from veritac_b200.CodeGen import gemmini_lowering
    return gemmini_lowering


def gemm(native, a, b, m, n, k, **kw):
    c = np.full(m * n, -2**31, dtype=np.int32)   # poison: every cell must be written
    native.i8gemm(np.ascontiguousarray(a), np.ascontiguousarray(b), c, m, n, k, **kw)
    return c


def test_spike_recorded_outputs_bit_exact(native, g, golden_gemmini):
    """The 24 matrices upstream Gemmini Spike produced, through the C ABI and through run_commands."""
    for case in golden_gemmini["spike_outputs"]:
        p = case["plan"]
        for mode in case["modes"]:
            a, b = go.raw_fill_inputs(mode["mode"], case["size_a"], case["size_b"])
            assert gemm(native, a, b, p["m"], p["n"], p["k"]).tolist() == mode["C"]
            got, _ = g.run_commands(commands_from_dicts(case["commands"]), p, a.tolist(), b.tolist())
            assert got == mode["C"]


def test_recorded_output_hashes(native, g, golden_gemmini):
    """30 recorded sha256(json.dumps(C)) of accepted programs, reproduced by run_commands on the GPU."""
    for run in golden_gemmini["recorded_hashes"]:
        p = run["plan"]
        cmds = commands_from_dicts(run["commands"])
        for case in run["cases"]:
            A, B = g.deterministic_inputs(p["m"], p["n"], p["k"], case["seed"], case["mode"])
            C, stats = g.run_commands(cmds, p, A, B)
            assert sha(C) == case["output_sha256"] and stats == case["stats"]


def test_compact_schedule_expands_and_runs(native, g, golden_schedule_ir):
    """A loop-form schedule goes through the adapter, the strict command objects and the GPU; the
    search controller's interpretation step reports it as matching the reference product."""
    from veritac_b200.specializations.gemmini_gemm import evaluation, schedule_ir

    p = golden_schedule_ir["programs"][0]
    plan = p["plan"]
    cmds = commands_from_dicts(schedule_ir.expand_program(p["program"], p["constants"]))
    A, B = g.deterministic_inputs(plan["m"], plan["n"], plan["k"], 11)
    C, stats = g.run_commands(cmds, plan, A, B)
    assert C == go.scalar_matmul(A, B, plan["m"], plan["n"], plan["k"])
    assert evaluation.interpret_commands(plan, cmds) == {"ran": True, "matches_reference": True}
    broken = cmds[:-2] + cmds[-1:]          # the last tile is never moved out
    got = evaluation.interpret_commands(plan, broken)
    assert got["ran"] is True and got["matches_reference"] is False and "error" in got
    assert evaluation.interpret_commands(plan, cmds, interpret_macs_limit=1000) == {
        "ran": False, "reason": "skipped: 65536 modeled MACs exceed the interpretation bound 1000"}


def test_learned_strategy_streams_on_the_gpu(native, g, golden_learned_streams):
    """14 streams from the reference's learned-strategy generators, executed here: same output hashes and
    stats as the reference's interpreter recorded, same refusal for the oversized batch."""
    for case in golden_learned_streams["cases"]:
        p = case["plan"]
        cmds = commands_from_dicts(case["commands"])
        for run in case["runs"]:
            A, B = g.deterministic_inputs(p["m"], p["n"], p["k"], run["seed"], run["mode"])
            if "error" in run:
                with pytest.raises(g.GemminiError) as info:
                    g.run_commands(cmds, p, A, B)
                assert str(info.value) == run["error"]
                continue
            C, stats = g.run_commands(cmds, p, A, B)
            assert sha(C) == run["output_sha256"] and stats == run["stats"], case["generator"]


def test_generator_streams_match_reference_interpreter(native, g, lowering, golden_gemmini):
    for e in golden_gemmini["generators"]:
        if "runs" not in e:
            continue
        plan, b = e["plan"], e["batch_rows"]
        cmds = g.gen_commands(plan) if b is None else lowering.gen_batched_reuse_b(plan, b)
        for run in e["runs"]:
            A, B = g.deterministic_inputs(plan["m"], plan["n"], plan["k"], run["seed"], run["mode"])
            assert sha(A) == run["a_sha256"] and sha(B) == run["b_sha256"]
            C, stats = g.run_commands(cmds, plan, A, B)
            assert sha(C) == run["output_sha256"] and stats == run["stats"]
            assert C == g.scalar_matmul(A, B, plan["m"], plan["n"], plan["k"])
            C2, stats2 = g.run_plan(plan, A, B, batch_rows=b)
            assert C2 == C and stats2 == stats


def test_reference_differential_cases(native, g):
    """tests/test_gemmini.py:52-75 of the reference: shapes x schedules x input modes."""
    cases = [((16, 16, 16), (("lcg", 7), ("max", 0), ("minmax", 0))),
             ((32, 32, 32), (("lcg", 1), ("lcg", 987654321), ("max", 0), ("minmax", 0))),
             ((48, 32, 64), (("lcg", 42), ("max", 0), ("minmax", 0))), ((64, 64, 64), (("lcg", 3), ("min", 0)))]
    for (m, n, k), modes in cases:
        for schedule in g.SUPPORTED_SCHEDULES:
            for mode, seed in modes:
                A, B = g.deterministic_inputs(m, n, k, seed, mode)
                plan = g.make_plan(m, n, k, schedule)
                C, stats = g.run_commands(g.gen_commands(plan), plan, A, B)
                assert C == go.scalar_matmul(A, B, m, n, k)
                assert stats["macs"] == m * n * k
    winner = g.optimize(48, 32, 64)["winner"]
    A, B = g.deterministic_inputs(48, 32, 64, 5)
    C, _ = g.run_commands(g.gen_commands(winner), winner, A, B)
    assert C == go.scalar_matmul(A, B, 48, 32, 64)


def test_config2_int8_64_cubed_partial_sums(native, g):
    """The 64^3 workload on the 4x4x4 tile grid, nonzero partial sums over the 4 K tiles."""
    rng = np.random.default_rng(20260917 + 2)
    a = rng.integers(-128, 128, 64 * 64, dtype=np.int8)
    b = rng.integers(-128, 128, 64 * 64, dtype=np.int8)
    want = go.matmul_exact(a, b, 64, 64, 64).reshape(-1)
    part = go.matmul_exact(a.reshape(64, 64)[:, :16].reshape(-1), b.reshape(64, 64)[:16].reshape(-1), 64, 64, 16)
    assert np.count_nonzero(part) > 0 and not np.array_equal(part.reshape(-1), want)
    for schedule in g.SUPPORTED_SCHEDULES:
        plan = g.make_plan(64, 64, 64, schedule)
        C, stats = g.run_commands(g.gen_commands(plan), plan, a, b)
        assert C.dtype == np.int32 and np.array_equal(C, want)
        assert (stats["overwrites"], stats["accumulates"]) == (256, 768)


@pytest.mark.parametrize("variant", [0, 1, 3, 4])
def test_shapes_rasters_variants(native, variant):
    rng = np.random.default_rng(11)
    shapes = [(16, 16, 16), (16, 80, 32), (80, 16, 32), (48, 32, 64), (128, 256, 128), (144, 272, 400),
              (256, 512, 384), (640, 768, 256), (1024, 1024, 1024), (2048, 16, 48), (16, 4096, 16)]
    for (m, n, k) in shapes:
        a = rng.integers(-128, 128, m * k, dtype=np.int8)
        b = rng.integers(-128, 128, k * n, dtype=np.int8)
        want = go.matmul_exact(a, b, m, n, k).reshape(-1)
        for raster, br in ((0, 1), (1, 1), (2, 3), (2, 64), (3, 1)):
            assert np.array_equal(gemm(native, a, b, m, n, k, variant=variant, raster=raster, batch_rows=br), want)


@pytest.mark.parametrize("variant", [0, 1, 3, 4])
def test_host_buffers_large_enough_for_the_corner_pipeline(native, variant):
    """From 2048 x 2048 outputs on, host-buffer calls bring B in by column blocks and return C by
    regions (pitched copies, kernels on sub-matrices)."""
    rng = np.random.default_rng(12)
    for (m, n, k) in ((2048, 2048, 32), (2320, 2576, 64), (4112, 2064, 48), (2064, 6160, 16)):
        a = rng.integers(-128, 128, m * k, dtype=np.int8)
        b = rng.integers(-128, 128, k * n, dtype=np.int8)
        want = go.matmul_exact(a, b, m, n, k).reshape(-1)
        assert np.array_equal(gemm(native, a, b, m, n, k, variant=variant), want)


def test_extreme_values_at_the_overflow_bound(native):
    """-128 * -128 * K and -128 * 127 * K at K = 8192 (|sum| = 2^27) and at the largest legal K."""
    for k in (8192, 131056):
        m, n = 32, 48
        for av, bv in ((-128, -128), (-128, 127), (127, 127)):
            a = np.full(m * k, av, dtype=np.int8)
            b = np.full(k * n, bv, dtype=np.int8)
            c = gemm(native, a, b, m, n, k)
            assert (c == av * bv * k).all()
    alt_a, alt_b = go.raw_fill_inputs("extrema", 64 * 8192, 8192 * 64)
    assert np.array_equal(gemm(native, alt_a, alt_b, 64, 64, 8192), go.matmul_exact(alt_a, alt_b, 64, 64, 8192).reshape(-1))


def test_device_resident_call_and_status(native):
    import torch
    rng = np.random.default_rng(5)
    m, n, k = 384, 512, 640
    a = rng.integers(-128, 128, (m, k), dtype=np.int8)
    b = rng.integers(-128, 128, (k, n), dtype=np.int8)
    dA, dB = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    dC = torch.full((m, n), -2**31, dtype=torch.int32, device="cuda")
    before = native.launch_count()
    native.i8gemm(dA, dB, dC, m, n, k, where=native.VT_DEVICE, stream=native.torch_stream())
    native.sync(0, native.torch_stream())
    assert native.launch_count() == before + 1
    assert np.array_equal(dC.cpu().numpy(), go.matmul_exact(a, b, m, n, k).astype(np.int32))


def test_shared_b_batch(native):
    """Batched B-reuse, small: independent A_i against one B."""
    rng = np.random.default_rng(9)
    batch, m, n, k = 5, 48, 64, 96
    a = rng.integers(-128, 128, (batch, m, k), dtype=np.int8)
    b = rng.integers(-128, 128, (k, n), dtype=np.int8)
    for acc_rows in (16, 32, 1024):
        c = np.full((batch, m, n), -2**31, dtype=np.int32)
        native.i8gemm_shared_b(a, b, c, batch, m, n, k, acc_rows=acc_rows)
        for i in range(batch):
            assert np.array_equal(c[i], go.matmul_exact(a[i], b, m, n, k).astype(np.int32))


def test_tile_program_for_streams_that_are_not_a_gemm(native, g):
    """Valid streams whose result is not the full product run tile by tile and still equal the
    sequential interpreter: K truncated to the first tile; and a stream that never accumulates."""
    m = n = k = 48
    A, B = g.deterministic_inputs(m, n, k, 77)
    plan = g.make_plan(m, n, k, "baseline")
    cmds = g.gen_commands(plan)
    for c in cmds:
        if c.kind == "preload":
            c.out_addr &= ~g.ACCUMULATE_BIT      # every K tile overwrites: C = last K tile's product
    want, want_stats = go.interpret(cmds, plan, A, B)
    got, stats = g.run_commands(cmds, plan, A, B)
    assert got == want and stats == want_stats and got != go.scalar_matmul(A, B, m, n, k)
    # same output tile moved out twice with different contents: the later mvout wins
    cmds = g.gen_commands(plan)
    first_mvout = next(i for i, c in enumerate(cmds) if c.kind == "mvout")
    dup = g.Mvout(16, cmds[first_mvout].acc_addr, 16, 16)      # tile (0,0)'s accumulator also lands on tile (0,1)
    cmds.insert(first_mvout + 1, dup)
    want, _ = go.interpret(cmds, plan, A, B)
    got, _ = g.run_commands(cmds, plan, A, B)
    assert got == want


def test_full_size_8192_cubed_properties(native):
    """The 8192^3 workload at full size, device resident: sampled rows against the exact product,
    the row-sum identity C*1 = A*(B*1) over every cell, poison fully overwritten, raster
    independence, and M-row sharding equals the unsharded result."""
    import torch
    M = N = K = 8192
    gen = torch.Generator(device="cuda").manual_seed(20260917 + 3)
    A = torch.randint(-128, 128, (M, K), dtype=torch.int8, device="cuda", generator=gen)
    B = torch.randint(-128, 128, (K, N), dtype=torch.int8, device="cuda", generator=gen)
    C = torch.full((M, N), -2**31, dtype=torch.int32, device="cuda")
    st = native.torch_stream()
    native.i8gemm(A, B, C, M, N, K, where=native.VT_DEVICE, stream=st)
    native.sync(0, st)
    rows = torch.randint(0, M, (48,), device="cuda", generator=gen)
    exact = (A[rows].double() @ B.double()).to(torch.int64)
    assert torch.equal(C[rows].to(torch.int64), exact)
    ones = B.to(torch.int64).sum(dim=1)                       # B * 1
    assert torch.equal(C.to(torch.int64).sum(dim=1), (A.to(torch.float64) @ ones.to(torch.float64)).to(torch.int64))
    C2 = torch.full((M, N), -2**31, dtype=torch.int32, device="cuda")
    native.i8gemm(A, B, C2, M, N, K, raster=native.VT_RASTER_BASELINE, where=native.VT_DEVICE, stream=st)
    native.sync(0, st)
    assert torch.equal(C, C2)
    from veritac_b200.sharding import row_shard
    C3 = torch.full((M, N), -2**31, dtype=torch.int32, device="cuda")
    for r in range(8):
        r0, r1 = row_shard(M, 8, r)
        native.i8gemm(A[r0:r1], B, C3[r0:r1], r1 - r0, N, K, where=native.VT_DEVICE, stream=st)
    native.sync(0, st)
    assert torch.equal(C, C3)


def test_host_buffers_equal_device_buffers_large(native):
    """The host-pointer entry point (row-block pipeline of copies and launches) at a multi-block size."""
    import torch
    rng = np.random.default_rng(21)
    m, n, k = 8192 + 256, 1024, 512
    a = rng.integers(-128, 128, (m, k), dtype=np.int8)
    b = rng.integers(-128, 128, (k, n), dtype=np.int8)
    c = np.full((m, n), -2**31, dtype=np.int32)
    native.i8gemm(a, b, c, m, n, k)
    want = (torch.from_numpy(a).cuda().double() @ torch.from_numpy(b).cuda().double()).to(torch.int32).cpu().numpy()
    assert np.array_equal(c, want)


def test_measure_controls_matches_reference_scoring(native, g, lowering):
    """The reference's tests/test_gemmini_evaluation.py:16-31 on the measured counterpart: a known
    batched stream is recognised as an existing control, gains nothing over the best one, and every
    control computes the same bits."""
    from veritac_b200.specializations.gemmini_gemm.evaluation import measure_controls
    plan = g.make_plan(32, 16, 16, "baseline")
    plan["accumulator_rows"] = 32
    a, b = go.deterministic_inputs(32, 16, 16, 3)
    result = measure_controls(plan, lowering.gen_batched_reuse_b(plan, 2), a, b, repeats=3)
    assert result["input_reduction_vs_baseline"] > 0
    assert result["input_reduction_vs_best_existing"] == 0
    assert result["beats_best_existing_objective"] is False
    assert "existing_batched_b_2" in result["exact_matches"]
    assert result["bit_exact"] is True and result["hardware_latency"]["candidate"] > 0
    assert [c["name"] for c in result["controls"]] == ["baseline", "existing_batched_b_1", "existing_batched_b_2"]
    with pytest.raises(ValueError, match="candidate failed"):
        measure_controls(g.make_plan(16, 16, 16, "baseline"), [g.Fence()], a[:256], b[:256])


def test_stream_order_holds_across_overlapped_launches(native):
    """The int8 kernels may be placed on the GPU while the kernel before them on the stream is still running
    and must not touch memory until it has completed.  A large fill of C runs right before each product with
    no synchronisation in between: if the product's stores did not wait, the fill would overwrite them."""
    import torch
    rng = np.random.default_rng(31)
    m, n, k = 4096, 4096, 64          # a short product behind a 64 MiB fill
    a = rng.integers(-128, 128, (m, k), dtype=np.int8)
    b = rng.integers(-128, 128, (k, n), dtype=np.int8)
    want = go.matmul_exact(a.reshape(-1), b.reshape(-1), m, n, k).reshape(m, n).astype(np.int32)
    dA, dB = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    dC = torch.empty((m, n), dtype=torch.int32, device="cuda")
    st = native.torch_stream()
    for variant in (0, 1, 3, 4):
        for rep in range(8):
            dC.fill_(-7 - rep)
            native.i8gemm(dA, dB, dC, m, n, k, variant=variant, where=native.VT_DEVICE, stream=st)
        native.sync(0, st)
        assert np.array_equal(dC.cpu().numpy(), want), variant
        # and a product whose input is the previous kernel's output: B2 is written by a copy kernel right before
        dB2 = torch.empty_like(dB)
        for rep in range(4):
            dB2.fill_(0)
            dB2.copy_(dB)
            native.i8gemm(dA, dB2, dC, m, n, k, variant=variant, where=native.VT_DEVICE, stream=st)
        native.sync(0, st)
        assert np.array_equal(dC.cpu().numpy(), want), variant


def _device_case(native, m, n, k, seed, variant=0, reps=2):
    """C of a device-resident call (poisoned first), checked on every cell against the exact product taken in
    float64 on the GPU (exact below 2^53); `reps` calls back to back."""
    import torch
    gen = torch.Generator(device="cuda").manual_seed(seed)
    A = torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda", generator=gen)
    B = torch.randint(-128, 128, (k, n), dtype=torch.int8, device="cuda", generator=gen)
    want = torch.empty((m, n), dtype=torch.int32, device="cuda")
    Bd = B.double()
    for r0 in range(0, m, 2048):
        want[r0:r0 + 2048] = (A[r0:r0 + 2048].double() @ Bd).to(torch.int32)
    st = native.torch_stream()
    for rep in range(reps):
        C = torch.full((m, n), -2**31, dtype=torch.int32, device="cuda")
        native.i8gemm(A, B, C, m, n, k, variant=variant, where=native.VT_DEVICE, stream=st)
        native.sync(0, st)
        assert torch.equal(C, want), (m, n, k, variant, rep)


@pytest.mark.parametrize("variant", [0, 3, 4])
def test_partial_rounds_of_the_pair_kernels(native, variant):
    """Shapes whose tiles do not fill whole rounds of the 74 CTA pairs, every cell checked: the 1024- and 2048-row
    shards of the 8192^3 problem (8 and 4 GPUs), fewer tiles than pairs, ragged edges, K not a multiple of the
    128-value block, long K."""
    shapes = [(1024, 8192, 8192), (2048, 8192, 8192), (1536, 4864, 4096), (512, 5376, 4096), (1000 - 8, 8192 - 48, 8192 + 48),
              (768, 3072, 32768), (256, 2560, 65536), (2048 + 16, 5120 + 16, 16384 + 16),
              (2048 - 16, 8192 + 32, 4096 + 16), (1280, 4352, 3072), (768, 7168, 2048)]
    for i, (m, n, k) in enumerate(shapes):
        _device_case(native, m, n, k, 20260917 + 40 + i, variant=variant)


def test_tile_shapes_and_rasters_give_the_same_bits(native):
    """The same inputs through 256 x 256 and 256 x 512 tiles, every raster: identical bits."""
    import torch
    gen = torch.Generator(device="cuda").manual_seed(20260917 + 60)
    m, n, k = 1024, 8192, 8192
    A = torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda", generator=gen)
    B = torch.randint(-128, 128, (k, n), dtype=torch.int8, device="cuda", generator=gen)
    st = native.torch_stream()
    outs = []
    for variant in (native.VT_I8_CTA_PAIR, native.VT_I8_CTA_PAIR_WIDE):
        for raster, br in ((0, 1), (1, 1), (2, 3), (3, 1)):
            C = torch.full((m, n), -2**31, dtype=torch.int32, device="cuda")
            native.i8gemm(A, B, C, m, n, k, variant=variant, raster=raster, batch_rows=br, where=native.VT_DEVICE, stream=st)
            native.sync(0, st)
            outs.append(C)
    assert all(torch.equal(outs[0], c) for c in outs[1:])


def test_batched_share_of_one_gpu_at_full_size(native):
    """One GPU's share of the batched B-reuse workload on eight GPUs: 32 x (1024 x 4096 . 4096 x 4096) through
    vt_i8gemm_shared_b, device resident: sampled rows of every A_i against the exact product, and the identity
    C.1 = A.(B.1) over every cell."""
    import torch
    batch, m, n, k = 32, 1024, 4096, 4096
    gen = torch.Generator(device="cuda").manual_seed(20260917 + 61)
    A = torch.randint(-128, 128, (batch * m, k), dtype=torch.int8, device="cuda", generator=gen)
    B = torch.randint(-128, 128, (k, n), dtype=torch.int8, device="cuda", generator=gen)
    C = torch.full((batch * m, n), -2**31, dtype=torch.int32, device="cuda")
    st = native.torch_stream()
    native.i8gemm_shared_b(A, B, C, batch, m, n, k, acc_rows=16, where=native.VT_DEVICE, stream=st)
    native.sync(0, st)
    rows = torch.cat([torch.randint(0, m, (4,), device="cuda", generator=gen) + i * m for i in range(batch)])
    assert torch.equal(C[rows].to(torch.int64), (A[rows].double() @ B.double()).to(torch.int64))
    ones = B.to(torch.int64).sum(dim=1)
    assert torch.equal(C.to(torch.int64).sum(dim=1), (A.to(torch.float64) @ ones.to(torch.float64)).to(torch.int64))


def test_host_buffers_8192_cubed_through_the_corner_pipeline(native):
    """The host-pointer call at the size the end-to-end figure is quoted on: B arrives in column blocks, C leaves
    in growing corner regions.  Sampled rows against the exact product and the row-sum identity over every cell."""
    import torch
    M = N = K = 8192
    gen = torch.Generator(device="cuda").manual_seed(20260917 + 62)
    A = torch.randint(-128, 128, (M, K), dtype=torch.int8, device="cuda", generator=gen)
    B = torch.randint(-128, 128, (K, N), dtype=torch.int8, device="cuda", generator=gen)
    hA, hB = A.cpu().pin_memory(), B.cpu().pin_memory()
    hC = torch.full((M, N), -2**31, dtype=torch.int32).pin_memory()
    native.i8gemm(hA, hB, hC, M, N, K, where=native.VT_HOST)
    C = hC.cuda()
    rows = torch.randint(0, M, (64,), device="cuda", generator=gen)
    assert torch.equal(C[rows].to(torch.int64), (A[rows].double() @ B.double()).to(torch.int64))
    ones = B.to(torch.int64).sum(dim=1)
    assert torch.equal(C.to(torch.int64).sum(dim=1), (A.to(torch.float64) @ ones.to(torch.float64)).to(torch.int64))


@pytest.mark.parametrize("stride_a,stride_b", [(0, 32), (1, 32), (16, 0), (16, 1), (33, 32), (16, 31), (0, 0)])
def test_load_strides_zero_one_and_beyond_a_row(native, g, stride_a, stride_b):
    """config_ld strides the reference's interpreter accepts (any stride_bytes >= 0): 0 repeats one row, 1 makes
    the rows of a tile overlap, more than a row skips rows.  The tile-program kernel must read exactly those rows;
    checked against the sequential interpreter."""
    from test_gemmini_host import _strided_stream
    plan, cmds = _strided_stream(stride_a, stride_b)
    A, B = g.deterministic_inputs(32, 32, 16, 9)
    want, want_stats = go.interpret(cmds, plan, A, B)
    got, stats = g.run_commands(cmds, plan, A, B)
    assert got == want and stats == want_stats


def test_rows_with_b_streamed_in_column_blocks(native):
    """One rank's step of the row-sharded job: A and C in pinned host memory, B staged block by block from host
    memory into dense device blocks (what rank 0 does before each broadcast), an event per block, one call that
    overlaps all of it.  Every cell against the exact product; ragged last block; a second call reuses the events."""
    import torch
    from veritac_b200.sharding import column_blocks
    gen = torch.Generator(device="cuda").manual_seed(20260917 + 70)
    st = native.torch_stream()
    for (m, n, k, nb) in ((1024, 8192, 8192, 8), (528, 2000 * 16 // 16 * 16 + 48, 1040, 5), (16, 16, 16, 1)):
        A = torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda", generator=gen)
        B = torch.randint(-128, 128, (k, n), dtype=torch.int8, device="cuda", generator=gen)
        want = (A.double() @ B.double()).to(torch.int32).cpu()
        hA, hB = A.cpu().pin_memory(), B.cpu().pin_memory()
        blocks = column_blocks(n, nb)
        bufs = [torch.empty((k, cols), dtype=torch.int8, device="cuda") for _c0, cols in blocks]
        events = [torch.cuda.Event() for _ in blocks]
        for rep in range(2):
            hC = torch.full((m, n), -2**31, dtype=torch.int32).pin_memory()
            for j, (c0, cols) in enumerate(blocks):
                native.i8_stage_b_block(bufs[j], hB, k, n, c0, cols, stream=st)
                events[j].record()
            if rep == 0:
                native.i8gemm_rows_streamed_b(hA, bufs, [c for _c0, c in blocks], events, hC, m, n, k)
            else:       # A already on the device, queued on the same stream before the blocks' events
                native.i8gemm_rows_streamed_b(A, bufs, [c for _c0, c in blocks], events, hC, m, n, k,
                                              a_where=native.VT_DEVICE)
            assert torch.equal(hC, want), (m, n, k, rep)
    with pytest.raises(native.NativeError):          # widths must add up to N
        native.i8gemm_rows_streamed_b(hA, bufs, [32], events, hC, 16, 16, 16)


def test_two_streams_joined_by_events(native):
    """Calls on one device must be ordered with one another on the GPU; two streams that hand over to each other
    through events are such an order.  int8 and fp32 calls alternate between two streams, each waiting for the
    other's last call; every result is checked (a race on the shared scratch, tickets or status word would show)."""
    import torch
    gen = torch.Generator(device="cuda").manual_seed(20260917 + 80)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    m, n, k = 1024, 8192, 2048
    A = torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda", generator=gen)
    B = torch.randint(-128, 128, (k, n), dtype=torch.int8, device="cuda", generator=gen)
    want = (A.double() @ B.double()).to(torch.int32)
    fa = torch.rand((16, 4096), device="cuda", generator=gen) * 2 - 1
    fb = torch.rand((4096, 4096), device="cuda", generator=gen) * 2 - 1
    fwant = fa.double() @ fb.double()
    outs_i, outs_f = [], []
    torch.cuda.synchronize()
    last = None
    for rep in range(6):
        stream = s1 if rep % 2 == 0 else s2
        with torch.cuda.stream(stream):
            if last is not None:
                stream.wait_event(last)
            C = torch.full((m, n), -2**31, dtype=torch.int32, device="cuda")
            F = torch.full((16, 4096), float("nan"), device="cuda")
            handle = int(stream.cuda_stream)
            native.i8gemm(A, B, C, m, n, k, variant=native.VT_I8_CTA_PAIR_WIDE if rep % 3 == 0 else 0,
                          where=native.VT_DEVICE, stream=handle)
            native.sgemm(fa, fb, F, 16, 4096, 4096, where=native.VT_DEVICE, stream=handle)
            last = torch.cuda.Event()
            last.record(stream)
            outs_i.append(C)
            outs_f.append(F)
    torch.cuda.synchronize()
    native.sync(0, int(s2.cuda_stream))
    for C in outs_i:
        assert torch.equal(C, want)
    for F in outs_f:
        assert float(torch.linalg.norm(F.double() - fwant) / torch.linalg.norm(fwant)) <= 1e-5


def test_host_rows_against_a_device_resident_b(native):
    """where = VT_HOST_AC_DEVICE_B: a rank's rows of A and C in host memory, the replicated B already on the device,
    produced on the stream the call is given (here a copy queued right before the call, standing in for the
    broadcast).  Plain and batched entry points, pinned and pageable host buffers, every cell against the exact product."""
    import torch
    gen = torch.Generator(device="cuda").manual_seed(20260917 + 71)
    st = native.torch_stream()
    for (m, n, k) in ((1024, 8192, 8192), (4096 + 16, 2048 + 16, 528), (16, 16, 16)):
        A = torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda", generator=gen)
        B = torch.randint(-128, 128, (k, n), dtype=torch.int8, device="cuda", generator=gen)
        want = (A.double() @ B.double()).to(torch.int32).cpu()
        hA = A.cpu().pin_memory()
        hC = torch.full((m, n), -2**31, dtype=torch.int32).pin_memory()
        dB = torch.zeros_like(B)
        dB.copy_(B, non_blocking=True)                       # still in flight on `st` when the call is made
        native.i8gemm(hA, dB, hC, m, n, k, where=native.VT_HOST_AC_DEVICE_B, stream=st)
        assert torch.equal(hC, want), (m, n, k)
        pageable = np.full((m, n), -2**31, dtype=np.int32)
        native.i8gemm(A.cpu().numpy(), dB, pageable, m, n, k, where=native.VT_HOST_AC_DEVICE_B, stream=st)
        assert np.array_equal(pageable, want.numpy())
    batch, m, n, k = 3, 256, 512, 384
    A = torch.randint(-128, 128, (batch * m, k), dtype=torch.int8, device="cuda", generator=gen)
    B = torch.randint(-128, 128, (k, n), dtype=torch.int8, device="cuda", generator=gen)
    hC = torch.full((batch * m, n), -2**31, dtype=torch.int32).pin_memory()
    native.i8gemm_shared_b(A.cpu().pin_memory(), B, hC, batch, m, n, k, acc_rows=32, where=native.VT_HOST_AC_DEVICE_B, stream=st)
    assert torch.equal(hC, (A.double() @ B.double()).to(torch.int32).cpu())
    with pytest.raises(native.NativeError):                 # no such form for the other `where` values
        native.i8gemm(hA, dB, hC, 16, 16, 16, where=7)
