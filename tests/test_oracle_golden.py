"""Pins the oracle (oracle/) to the reference's own golden vectors before anything trusts it."""
import ctypes
import hashlib
import json
import subprocess
import sys

import numpy as np
import pytest

import gemmini_oracle as go
import loopnest_oracle as lo
from conftest import STUB


def sha(obj):
    return hashlib.sha256(json.dumps(obj).encode()).hexdigest()


def test_raw_inputs_match_reference_streams(golden_gemmini):
    for case in golden_gemmini["spike_outputs"]:
        for mode in case["modes"]:
            a, b = go.raw_fill_inputs(mode["mode"], case["size_a"], case["size_b"])
            assert hashlib.sha256(a.tobytes()).hexdigest() == mode["a_sha256"]
            assert hashlib.sha256(b.tobytes()).hexdigest() == mode["b_sha256"]


def test_spike_recorded_outputs(golden_gemmini):
    """24 full int32 matrices produced by upstream Gemmini Spike: the exact product and the
    sequential interpreter both reproduce every cell."""
    n = 0
    for case in golden_gemmini["spike_outputs"]:
        p = case["plan"]
        for mode in case["modes"]:
            a, b = go.raw_fill_inputs(mode["mode"], case["size_a"], case["size_b"])
            want = mode["C"]
            assert go.matmul_exact(a, b, p["m"], p["n"], p["k"]).reshape(-1).tolist() == want
            got, _ = go.interpret(case["commands"], p, a.tolist(), b.tolist())
            assert got == want
            n += 1
    assert n == 24


def test_recorded_output_hashes(golden_gemmini):
    """30 sha256(json.dumps(C)) recorded by the reference for accepted blind-search programs."""
    n = 0
    for run in golden_gemmini["recorded_hashes"]:
        p = run["plan"]
        for case in run["cases"]:
            a, b = go.deterministic_inputs(p["m"], p["n"], p["k"], case["seed"], case["mode"])
            got, stats = go.interpret(run["commands"], p, a.tolist(), b.tolist())
            assert go.output_sha256(got) == case["output_sha256"]
            assert stats == case["stats"]
            assert go.scalar_matmul(a, b, p["m"], p["n"], p["k"]) == got
            n += 1
    assert n == 30


def test_deterministic_inputs(golden_gemmini):
    for d in golden_gemmini["deterministic_inputs"]:
        a, b = go.deterministic_inputs(*d["args"])
        assert sha(a.tolist()) == d["a_sha256"] and sha(b.tolist()) == d["b_sha256"]
        assert a[:8].tolist() == d["a_head"] and b[:8].tolist() == d["b_head"]
    with pytest.raises(ValueError):
        go.deterministic_inputs(16, 16, 16, 1, "nope")


def test_lcg_jump_ahead_equals_plain_loop():
    long = go._lcg_states(10000, 12345)
    x, plain = 12345, []
    for _ in range(10000):
        x = (1103515245 * x + 12345) & 0xFFFFFFFF
        plain.append(x)
    assert long.tolist() == plain


def test_exact_product_equals_literal_loops():
    rng = np.random.default_rng(3)
    a = rng.integers(-128, 128, 16 * 48).tolist()
    b = rng.integers(-128, 128, 48 * 32).tolist()
    assert go.scalar_matmul(a, b, 16, 32, 48) == go.scalar_matmul_loops(a, b, 16, 32, 48)


def test_c_scalar_and_tiled_refs(liboracle):
    rng = np.random.default_rng(4)
    for (m, n, k) in ((16, 16, 16), (48, 32, 64), (64, 80, 32)):
        a = rng.integers(-128, 128, m * k, dtype=np.int8)
        b = rng.integers(-128, 128, k * n, dtype=np.int8)
        want = go.matmul_exact(a, b, m, n, k).astype(np.int32).reshape(-1)
        c1 = np.full(m * n, -1, dtype=np.int32)
        c2 = np.full(m * n, -1, dtype=np.int32)
        liboracle.oracle_i8_scalar_ref(a.ctypes.data, b.ctypes.data, c1.ctypes.data, m, n, k)
        liboracle.oracle_i8_tiled_ref(a.ctypes.data, b.ctypes.data, c2.ctypes.data, m, n, k, 0, m)
        assert np.array_equal(c1, want) and np.array_equal(c2, want)
    # worst case magnitudes: -128 * -128 * K
    m, n, k = 16, 16, 8192
    a = np.full(m * k, -128, dtype=np.int8)
    b = np.full(k * n, -128, dtype=np.int8)
    c = np.zeros(m * n, dtype=np.int32)
    liboracle.oracle_i8_tiled_ref(a.ctypes.data, b.ctypes.data, c.ctypes.data, m, n, k, 0, m)
    assert (c == 2**27).all()


def test_c_lcg_inputs(liboracle, golden_gemmini):
    d = golden_gemmini["deterministic_inputs"][1]
    m, n, k, seed, _ = d["args"]
    a = np.empty(m * k, dtype=np.int8)
    b = np.empty(k * n, dtype=np.int8)
    liboracle.oracle_i8_lcg_inputs(a.ctypes.data, a.size, b.ctypes.data, b.size, ctypes.c_uint32(seed))
    assert sha(a.tolist()) == d["a_sha256"] and sha(b.tolist()) == d["b_sha256"]


def _check(value):
    proc = subprocess.run([sys.executable, str(STUB)], input=json.dumps(value) + "\n", text=True, capture_output=True,
                          timeout=30)
    assert proc.returncode == 0
    return json.loads(proc.stdout)


def test_plan_checker_stub_boundary_cases():
    """The cases the reference's tests/test_gemmini_checker.py:26-62 puts to the Lean executable."""
    def plan(**ch):
        p = dict(m=32, n=32, k=32, dim=16, scratchpad_rows=32, accumulator_rows=32, schedule="reuse_b")
        p.update(ch)
        return p

    ok = _check(plan())
    assert ok["accepted"] is True and ok["plan"] == plan()
    rej = _check(plan(accumulator_rows=31))
    assert rej["accepted"] is False and "plan" not in rej
    assert _check(plan(schedule="baseline", accumulator_rows=16))["accepted"] is True
    assert _check(plan(schedule="baseline", accumulator_rows=15))["accepted"] is False
    assert _check(plan(scratchpad_rows=31))["accepted"] is False
    for ch in (dict(m=0), dict(n=0), dict(k=0), dict(dim=0), dict(m=31), dict(n=17), dict(k=33), dict(k=131072),
               dict(schedule="unknown")):
        out = _check(plan(**ch))
        assert out["accepted"] is False and "plan" not in out
    assert _check(plan(k=131056))["accepted"] is True
    for name in ("m", "n", "k", "dim", "scratchpad_rows", "accumulator_rows"):
        for value in (-1, 0.5, True, None, "32", [], {}):
            assert _check(plan(**{name: value}))["accepted"] is False
        missing = plan()
        del missing[name]
        assert _check(missing)["accepted"] is False
    for value in (None, [], "plan", 42):
        assert _check(value)["accepted"] is False
    proc = subprocess.run([sys.executable, str(STUB)], input="{broken\n", text=True, capture_output=True, timeout=30)
    assert proc.returncode == 0 and json.loads(proc.stdout)["accepted"] is False


def test_plan_legal_matches_stub():
    for ch in ({}, {"accumulator_rows": 31}, {"k": 131072}, {"k": 131056}, {"scratchpad_rows": 31}):
        p = dict(m=32, n=32, k=32, dim=16, scratchpad_rows=32, accumulator_rows=32, schedule="reuse_b")
        p.update(ch)
        assert go.plan_legal(p)[0] == _check(p)["accepted"]


def test_loopnest_semantics_2x2_block():
    """The reference's tests/test_matmul.py:59-76: a 2x2 block inside a 4^3 nest gives [[19,22],[43,50]]."""
    store = {n: np.zeros(4 * lo.STRIDE) for n in "ABC"}
    store["A"][[0, 1, 1000, 1001]] = [1, 2, 3, 4]
    store["B"][[0, 1, 1000, 1001]] = [5, 6, 7, 8]
    lo.execute(lo.matmul_stmt(4, 4, 4), store)
    assert store["C"][[0, 1, 1000, 1001]].tolist() == [19, 22, 43, 50]


def test_tactics_pins(golden_cpu_gemm):
    """tests/test_matmul.py:136-155 and tests/test_soundness.py:41-86 of the reference."""
    t = lo.apply_tactics(lo.matmul_stmt(256, 256, 256), [
        {"kind": "tile", "vars": ["i0"], "int_params": [32]}, {"kind": "tile", "vars": ["i1"], "int_params": [32]},
        {"kind": "parallel", "vars": ["i0_outer"], "int_params": []}])
    assert t["var"] == "i0_outer" and t["ann"] == "parallel" and t["body"]["var"] == "i0_inner"
    assert golden_cpu_gemm["tactic_pins"] == {"outer_var": "i0_outer", "outer_ann": "parallel",
                                              "inner_var": "i0_inner"}
    with pytest.raises(lo.TacticError):
        lo.tile(lo.matmul_stmt(10, 10, 10), "i0", 3)          # non-dividing tile
    with pytest.raises(lo.TacticError):
        lo.parallel(lo.matmul_stmt(8, 8, 8), "i2")            # reduction loop
    with pytest.raises(lo.TacticError):
        lo.vectorize(lo.matmul_stmt(8, 8, 8), "i0")           # not innermost
    # tiling and reordering preserve the meaning of the nest
    a, b = lo.runner_operands(8, 8, 8)
    def run(stmt):
        store = {"A": np.zeros(8 * lo.STRIDE), "B": np.zeros(8 * lo.STRIDE), "C": np.zeros(8 * lo.STRIDE)}
        for i in range(8):
            store["A"][i * lo.STRIDE:i * lo.STRIDE + 8] = a[i]
            store["B"][i * lo.STRIDE:i * lo.STRIDE + 8] = b[i]
        lo.execute(stmt, store)
        return np.stack([store["C"][i * lo.STRIDE:i * lo.STRIDE + 8] for i in range(8)])
    sched = [{"kind": "tile", "vars": ["i0"], "int_params": [4]}, {"kind": "tile", "vars": ["i1"], "int_params": [2]},
             {"kind": "reorder", "vars": ["i1_inner", "i2"], "int_params": []},
             {"kind": "vectorize", "vars": ["i1_inner"], "int_params": []},
             {"kind": "parallel", "vars": ["i0_outer"], "int_params": []}]
    assert np.array_equal(run(lo.matmul_stmt(8, 8, 8)), a @ b)
    assert np.array_equal(run(lo.apply_tactics(lo.matmul_stmt(8, 8, 8), sched)), a @ b)


def test_c_loop_nests_agree_with_float64(liboracle, golden_cpu_gemm):
    """The C restatements of the generated nests reproduce the cells the reference's runner printed."""
    for run in golden_cpu_gemm["benchmark_matmul"]:
        M, K, N = run["M"], run["K"], run["N"]
        a, b = lo.runner_operands(M, K, N)
        c = np.zeros((M, N))
        fn = liboracle.oracle_dgemm_tuned if run["schedule"] else liboracle.oracle_dgemm_naive
        fn(a.ctypes.data, b.ctypes.data, c.ctypes.data, M, N, K)
        cells = [c[0, 0], c[1, 0], c[M - 1, 0], c[M - 1, N - 1]]
        assert cells == run["c_first_values"] == run["np_first_values"] and run["correct"] is True
        assert lo.runner_reference_cells(M, K, N) == run["np_first_values"]
        a32, b32 = a.astype(np.float32), b.astype(np.float32)
        c32 = np.zeros((M, N), dtype=np.float32)
        fn32 = liboracle.oracle_sgemm_tuned if run["schedule"] else liboracle.oracle_sgemm_naive
        fn32(a32.ctypes.data, b32.ctypes.data, c32.ctypes.data, M, N, K)
        assert np.array_equal(c32.astype(np.float64), c)  # small integers: fp32 is exact too


def test_c_restatement_equals_reference_generated_c(liboracle):
    """oracle/_ref holds C printed by the reference's own, unmodified emitter (built by
    oracle/build_ref.py where the reference tree exists).  The restated nests must reproduce its
    result bit for bit on uniform random doubles: same loop order, same arithmetic."""
    from conftest import REPO
    ref_dir = REPO / "oracle" / "_ref"
    libs = sorted(ref_dir.glob("matmul_256_*.so"))
    if not libs:
        pytest.skip("oracle/_ref not built (no reference tree on this machine)")
    rng = np.random.default_rng(8)
    M = N = K = 256
    a = rng.random((M, K)) * 2 - 1
    b = rng.random((K, N)) * 2 - 1
    for lib in libs:
        fn = ctypes.CDLL(str(lib)).matmul
        fn.argtypes = [ctypes.c_void_p] * 3
        # the reference's layout: row stride 1000 doubles
        A = np.zeros(M * lo.STRIDE)
        B = np.zeros(K * lo.STRIDE)
        C = np.zeros(M * lo.STRIDE)
        A.reshape(M, lo.STRIDE)[:, :K] = a
        B.reshape(K, lo.STRIDE)[:, :N] = b
        fn(A.ctypes.data, B.ctypes.data, C.ctypes.data)
        got = C.reshape(M, lo.STRIDE)[:, :N]
        want = np.zeros((M, N))
        mine = liboracle.oracle_dgemm_tuned if "readme" in lib.name else liboracle.oracle_dgemm_naive
        mine(np.ascontiguousarray(a).ctypes.data, np.ascontiguousarray(b).ctypes.data, want.ctypes.data, M, N, K)
        assert np.array_equal(got, want), lib.name
        assert np.allclose(got, a @ b, rtol=0, atol=1e-11)
