"""Host-side logic of the cpu_gemm drop-in: parser, emitter text against the reference's, the GEMM
recogniser, the host compile-and-run helper, the catalog and the import aliases.  No GPU."""
import hashlib
import sys

import pytest

import loopnest_oracle as lo
from veritac_b200.specializations.cpu_gemm import emit_c, lower, recognise, runner


def test_emitter_text_is_the_references(golden_cpu_gemm):
    for name, case in golden_cpu_gemm["emit_function"].items():
        text = emit_c.emit_function("matmul", lower.parse_stmt(case["stmt"]), [("A", 1), ("B", 2)], [("C", 3)])
        assert hashlib.sha256(text.encode()).hexdigest() == case["sha256"], name
        if case["text"] is not None:
            assert text == case["text"]
    h = golden_cpu_gemm["emit_test_harness"]
    assert emit_c.emit_test_harness("f", [("A", 4)], [("C", 5)], "    A[0] = 1;") == h["with_init"]
    assert emit_c.emit_test_harness("f", [("A", 4), ("B", 1)], [("C", 5), ("D", 1)]) == h["two_each"]


def test_pragma_guard():
    nest = lower.parse_stmt(lo.matmul_stmt(8, 8, 8))
    assert emit_c.writes_local_to("i0", nest) and emit_c.writes_local_to("i1", nest)
    assert not emit_c.writes_local_to("i2", nest)
    red = lo.matmul_stmt(8, 8, 8)["body"]["body"]
    red["ann"] = "parallel"
    assert "parallel suppressed" in emit_c.emit_stmt(lower.parse_stmt(red))
    red["ann"] = "vectorize"
    assert "simd suppressed" in emit_c.emit_stmt(lower.parse_stmt(red))
    assert emit_c.flat_index_expr("X", []) == "0"


def test_parser_errors_and_defaults():
    with pytest.raises(ValueError):
        lower.parse_stmt({"tag": "while"})
    with pytest.raises(ValueError):
        lower.parse_expr({"tag": "sub"})
    loop = lower.parse_stmt({"tag": "loop", "var": "i", "lo": lo.lit(0), "hi": lo.lit(2), "body": {"tag": "skip"}})
    assert loop.annotation == "none" and isinstance(loop.body, lower.CSkip)
    assert lower.parse_expr({"tag": "lit", "val": "7"}) == lower.CLit(7)


def test_recogniser_accepts_every_schedule_of_the_matmul():
    for M, K, N in ((256, 256, 256), (64, 96, 32)):
        base = lo.matmul_stmt(M, K, N)
        info = recognise.recognise_matmul(lower.parse_stmt(base), M, K, N)
        assert [r for _, _, _, r in info["loops"]] == ["i", "j", "k"]
        tuned = lo.apply_tactics(base, lo.README_SCHEDULE)
        info = recognise.recognise_matmul(lower.parse_stmt(tuned), M, K, N)
        assert [(v, r) for v, _, _, r in info["loops"]] == [("i0_outer", "i"), ("i0_inner", "i"), ("i1_outer", "j"),
                                                            ("i2", "k"), ("i1_inner", "j")]
    deep = lo.apply_tactics(lo.matmul_stmt(64, 64, 64), [
        {"kind": "tile", "vars": ["i2"], "int_params": [16]}, {"kind": "tile", "vars": ["i2_inner"], "int_params": [4]},
        {"kind": "reorder", "vars": ["i1", "i2_outer"], "int_params": []},
        {"kind": "reorder", "vars": ["i0", "i2_outer"], "int_params": []}])
    recognise.recognise_matmul(lower.parse_stmt(deep), 64, 64, 64)


def test_recogniser_refuses_what_is_not_the_gemm():
    P = lower.parse_stmt
    with pytest.raises(recognise.NotAMatmul):      # sizes disagree with the nest
        recognise.recognise_matmul(P(lo.matmul_stmt(32, 32, 32)), 32, 32, 64)
    with pytest.raises(recognise.NotAMatmul):      # M, K, N swapped
        recognise.recognise_matmul(P(lo.matmul_stmt(16, 32, 48)), 16, 48, 32)
    bad = lo.matmul_stmt(8, 8, 8)
    bad["body"]["body"]["body"]["val"]["right"]["right"]["indices"] = [lo.var("i1"), lo.var("i2")]  # B[j,k]
    with pytest.raises(recognise.NotAMatmul):
        recognise.recognise_matmul(P(bad), 8, 8, 8)
    rep = {"tag": "loop", "var": "t", "lo": lo.lit(0), "hi": lo.lit(2), "ann": "none", "body": lo.matmul_stmt(8, 8, 8)}
    with pytest.raises(recognise.NotAMatmul):      # an extra loop repeats the accumulation
        recognise.recognise_matmul(P(rep), 8, 8, 8)
    off = lo.matmul_stmt(8, 8, 8)
    off["lo"] = lo.lit(1)
    with pytest.raises(recognise.NotAMatmul):
        recognise.recognise_matmul(P(off), 8, 8, 8)
    seq = {"tag": "seq", "s1": lo.matmul_stmt(8, 8, 8), "s2": {"tag": "skip"}}
    with pytest.raises(recognise.NotAMatmul):
        recognise.recognise_matmul(P(seq), 8, 8, 8)
    halved = lo.matmul_stmt(8, 8, 8)
    halved["body"]["body"]["body"]["indices"][0] = {"tag": "mul", "left": lo.var("i0"), "right": lo.lit(2)}
    with pytest.raises(recognise.NotAMatmul):
        recognise.recognise_matmul(P(halved), 8, 8, 8)
    with pytest.raises(RuntimeError):               # the drop-in entry point reports it as a run failure
        runner.benchmark_matmul(seq, 8, 8, 8)
    with pytest.raises(ValueError):
        runner.benchmark_matmul({"tag": "bogus"}, 8, 8, 8)


def test_compile_and_run_2x2_block():
    """The reference's tests/test_matmul.py:59-94 through this package's emitter and host compiler."""
    code = emit_c.emit_function("matmul", lower.parse_stmt(lo.matmul_stmt(4, 4, 4)),
                                [("A", 4000000), ("B", 4000000)], [("C", 4000000)]) + r"""
int main(void) {
    double* A = calloc(4000000, sizeof(double));
    double* B = calloc(4000000, sizeof(double));
    double* C = calloc(4000000, sizeof(double));
    A[0]=1; A[1]=2; A[1000]=3; A[1001]=4;
    B[0]=5; B[1]=6; B[1000]=7; B[1001]=8;
    matmul(A, B, C);
    printf("%g %g %g %g\n", C[0], C[1], C[1000], C[1001]);
    return 0;
}
"""
    out, elapsed = runner.compile_and_run(code)
    assert out.split() == ["19", "22", "43", "50"] and elapsed >= 0
    with pytest.raises(RuntimeError):
        runner.compile_and_run("int main(void) { return 3; }")
    with pytest.raises(RuntimeError):
        runner.compile_and_run("this is not C")


def test_operand_pattern_matches_reference_cells(golden_cpu_gemm):
    for run in golden_cpu_gemm["benchmark_matmul"]:
        M, K, N = run["M"], run["K"], run["N"]
        a, b = runner.matmul_operands(M, K, N, dtype="float64")
        c = a @ b
        assert [c[0, 0], c[1, 0], c[M - 1, 0], c[M - 1, N - 1]] == run["np_first_values"]


def test_catalog_imports_no_runtime():
    import subprocess
    code = ("import sys; sys.path.insert(0, %r); from veritac_b200.specializations import catalog; "
            "ids=[d['id'] for d in catalog.list_specializations()]; "
            "assert ids == ['cpu_gemm', 'gemmini_gemm'], ids; "
            "assert 'numpy' not in sys.modules and 'torch' not in sys.modules; print('ok')") % sys.path[0]
    from conftest import REPO
    r = subprocess.run([sys.executable, "-c", code.replace(repr(sys.path[0]), repr(str(REPO)))], capture_output=True,
                       text=True)
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stderr


def test_catalog_descriptions_and_paths():
    from conftest import REPO
    from veritac_b200.specializations import catalog
    keys = {"schema_version", "id", "status", "computation", "target", "implementation", "formal_sources",
            "entrypoints", "proof_scope", "boundaries", "evidence"}
    for name in ("cpu_gemm", "gemmini_gemm"):
        d = catalog.describe(name)
        assert set(d) == keys and d["schema_version"] == 1 and d["id"] == name
        for rel in d["implementation"] + d["evidence"]:
            assert (REPO / rel).exists(), rel
    for bad in ("", "Bad", "../x", 3, "nope"):
        with pytest.raises(ValueError):
            catalog.describe(bad)


def test_old_import_paths_are_the_same_modules():
    import veritac_b200
    from veritac_b200.CodeGen import emit_c as e1, gemmini as g1, gemmini_lowering as l1, lower as w1, runner as r1
    from veritac_b200.specializations.cpu_gemm import emit_c as e2, lower as w2, runner as r2
    from veritac_b200.specializations.gemmini_gemm import backend as g2, lowering as l2
    assert (e1 is e2) and (g1 is g2) and (l1 is l2) and (w1 is w2) and (r1 is r2)
    veritac_b200.install_aliases()
    from CodeGen import runner as top
    from specializations.cpu_gemm import runner as top2
    assert top is r2 and top2 is r2


def test_demo_scheduled_nest_is_what_the_tactics_produce():
    """The demo's directly-built README nest equals the nest the tactic restatement derives."""
    from veritac_b200.examples import gemm_demo
    for (M, K, N) in ((256, 256, 256), (64, 96, 128)):
        assert gemm_demo.naive_matmul_stmt(M, K, N) == lo.matmul_stmt(M, K, N)
        assert gemm_demo.readme_scheduled_stmt(M, K, N) == lo.apply_tactics(lo.matmul_stmt(M, K, N), lo.README_SCHEDULE)
    with pytest.raises(ValueError):
        gemm_demo.readme_scheduled_stmt(48, 32, 32)


def test_agent_loop_applies_verified_tactics_and_skips_refused_ones(golden_cpu_gemm, tmp_path, monkeypatch):
    """The verify-and-apply loop of the mock LLM demo (reference examples/llm_gemm_demo.py:260-333) against the
    tactic verifier's command-line contract (`veritac --json`, Main.lean:697-745; the stub restates the tactics).
    The fixed five-tactic proposal list turns the naive nest into the README-scheduled one; a proposal the verifier
    refuses leaves the nest as it was and the walk goes on; without the executable the loop fails closed."""
    from veritac_b200.examples import llm_gemm_demo as demo
    from veritac_b200.examples.gemm_demo import naive_matmul_stmt, readme_scheduled_stmt
    from veritac_b200.specializations.cpu_gemm.lower import parse_stmt
    from veritac_b200.specializations.cpu_gemm.recognise import recognise_matmul
    from veritac_b200.specializations.cpu_gemm.runner import schedule_hint

    lines = []
    schedule, final, refused = demo.run_agent(naive_matmul_stmt(64, 64, 64), demo.MockProposer(demo.mock_schedule()),
                                              log=lines.append)
    assert [t["kind"] for t in schedule] == ["tile", "tile", "reorder", "vectorize", "parallel"] and not refused
    assert final == readme_scheduled_stmt(64, 64, 64)
    assert any("proposer is done" in x for x in lines)
    hint = schedule_hint(recognise_matmul(parse_stmt(final), 64, 64, 64))
    assert (hint["tile_m"], hint["tile_n"], hint["parallel"], hint["vectorize"]) == (32, 32, ["i0_outer"], ["i1_inner"])
    assert schedule_hint(recognise_matmul(parse_stmt(naive_matmul_stmt(64, 64, 64)), 64, 64, 64))["variant"] is None

    # a tile size that does not divide the extent is refused; the remaining proposals still apply
    bad = [demo._tactic("tile", "i0", size=48)] + demo.mock_schedule()
    schedule, final, refused = demo.run_agent(naive_matmul_stmt(64, 64, 64), demo.MockProposer(bad), max_steps=10,
                                              log=lines.append)
    assert len(refused) == 1 and refused[0][0]["int_params"] == [48] and len(schedule) == 5
    assert final == readme_scheduled_stmt(64, 64, 64)
    # the step limit ends the walk early
    schedule, final, _ = demo.run_agent(naive_matmul_stmt(64, 64, 64), demo.MockProposer(demo.mock_schedule()),
                                        max_steps=2, log=lines.append)
    assert len(schedule) == 2
    # fail closed without the verifier
    monkeypatch.setenv("VERITAC_BIN", str(tmp_path / "missing"))
    with pytest.raises(FileNotFoundError, match="VeriTac binary not found"):
        demo.call_lean(naive_matmul_stmt(16, 16, 16), [])
