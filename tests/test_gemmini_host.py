"""Host-side logic of the gemmini_gemm drop-in against fixtures generated from the reference:
plan validation texts, generators, modeled counts, inputs, optimize, the fail-closed gate and the
symbolic replay (errors and stats).  No GPU is touched: everything here ends before execution."""
import hashlib
import json
from unittest import mock

import pytest

from conftest import commands_from_dicts
from veritac_b200.CodeGen import gemmini as g
from veritac_b200.CodeGen import gemmini_lowering as lowering

BIN_MISSING = "/nonexistent/veritac/gemmini_check"


def sha(obj):
    return hashlib.sha256(json.dumps(obj).encode()).hexdigest()


def test_constants_match_reference():
    assert (g.DIM, g.SCRATCHPAD_ROWS, g.ACC_ROWS, g.ELEM_MIN, g.ELEM_MAX) == (16, 16384, 1024, -128, 127)
    assert g.GARBAGE_ADDR == 0xFFFFFFFF and g.ACC_BASE_ADDR == 0xE0000000
    assert g.SUPPORTED_SCHEDULES == ("baseline", "reuse_b")


def test_validate_plan_verdicts_and_reasons(golden_gemmini):
    for v in golden_gemmini["validate_plan"]:
        ok, reason = g.validate_plan(v["plan"])
        assert (ok, reason) == (v["ok"], v["reason"]), v["plan"]


def test_make_plan_minimum_capacities():
    p = g.make_plan(32, 32, 32, g.SCHEDULE_BASELINE)
    assert (p["dim"], p["scratchpad_rows"], p["accumulator_rows"]) == (16, 32, 16)
    assert g.required_resources(p) == (32, 16)
    assert g.make_plan(48, 32, 64, g.SCHEDULE_REUSE_B)["accumulator_rows"] == 48
    for schedule in g.SUPPORTED_SCHEDULES:
        for shape in ((16, 16, 16), (32, 32, 32), (48, 32, 64)):
            assert g.validate_plan(g.make_plan(*shape, schedule)) == (True, "ok")


def test_generators_hashes_counts_and_replay_stats(golden_gemmini):
    for e in golden_gemmini["generators"]:
        plan, b = e["plan"], e["batch_rows"]
        if "value_error" in e:
            with pytest.raises(ValueError):
                lowering.gen_batched_reuse_b(plan, b)
            continue
        cmds = g.gen_commands(plan) if b is None else lowering.gen_batched_reuse_b(plan, b)
        assert lowering.command_hash(cmds) == e["command_sha256"]
        assert g.modeled_counts(cmds) == e["counts"]
        replay = g._Replay(plan)
        if "error" in e:
            with pytest.raises(g.GemminiError) as info:
                for c in cmds:
                    replay.step(c)
            assert str(info.value) == e["error"]
            continue
        for c in cmds:
            replay.step(c)
        replay.finish()
        assert replay.stats == e["runs"][0]["stats"]
        got = g._plain_gemm_raster(replay.tiles, plan["m"], plan["n"], plan["k"])
        it, jt = plan["m"] // 16, plan["n"] // 16
        if it == 1 or jt == 1:
            assert got in ("baseline", "reuse_b")      # orders coincide on a single row / column of tiles
        elif b is not None:
            # the batched lowering moves tiles out column by column, like reuse_b, with fewer rows live
            assert got == "reuse_b" and replay.max_acc_base // 16 + 1 == min(b, it)
        else:
            assert got == plan["schedule"]


def test_run_plan_closed_form_stats(golden_gemmini):
    """run_plan's analytic stats equal the interpreter's for every generator stream."""
    for e in golden_gemmini["generators"]:
        if "runs" not in e:
            continue
        plan, b = e["plan"], e["batch_rows"]
        it, jt, kt = plan["m"] // 16, plan["n"] // 16, plan["k"] // 16
        b_loads = (jt * kt * -(-it // b)) if b else (it * jt * kt if plan["schedule"] == "baseline" else jt * kt)
        stats = {"instructions": 4 + b_loads + 3 * it * jt * kt + it * jt + 1, "macs": it * jt * kt * 4096,
                 "overwrites": it * jt * 16, "accumulates": it * jt * (kt - 1) * 16}
        assert stats == e["runs"][0]["stats"]


def test_checked_request_streams(golden_gemmini):
    for r in golden_gemmini["checked_requests"]:
        cmds = g.serialize_commands(g.gen_commands(r["plan"]))
        assert len(cmds) == r["n_commands"] and sha(cmds) == r["commands_sha256"]
    assert len(g.gen_commands(g.make_plan(64, 64, 64, "baseline"))) == 277
    assert len(g.gen_commands(g.make_plan(64, 64, 64, "reuse_b"))) == 229


def test_command_structure_counts():
    base = g.modeled_counts(g.gen_commands(g.make_plan(32, 32, 32, g.SCHEDULE_BASELINE)))
    assert (base["mvin_A"], base["mvin_B"], base["mvout"], base["fence"]) == (8, 8, 4, 1)
    reuse = g.modeled_counts(g.gen_commands(g.make_plan(32, 32, 32, g.SCHEDULE_REUSE_B)))
    assert (reuse["mvin_A"], reuse["mvin_B"], reuse["mvout"], reuse["fence"]) == (8, 4, 4, 1)
    assert reuse["dma_bytes"] < base["dma_bytes"]
    # docs/gemmini_gemm.md:170-179 of the reference: modeled input bytes baseline -> reuse_b
    for shape, want in (((32, 32, 32), (4096, 3072)), ((64, 64, 64), (32768, 20480)), ((48, 32, 64), (12288, 8192)),
                        ((16, 48, 32), (3072, 3072))):
        got = tuple(g.modeled_counts(g.gen_commands(g.make_plan(*shape, s)))["dma_in_elems_int8"]
                    for s in g.SUPPORTED_SCHEDULES)
        assert got == want
    plan = g.make_plan(48, 16, 32, "baseline")
    plan["accumulator_rows"] = 32
    assert g.modeled_counts(lowering.gen_batched_reuse_b(plan, 2))["mvin_B"] == 4


def test_deterministic_inputs(golden_gemmini):
    for d in golden_gemmini["deterministic_inputs"]:
        a, b = g.deterministic_inputs(*d["args"])
        assert sha(a) == d["a_sha256"] and sha(b) == d["b_sha256"]
    with pytest.raises(ValueError):
        g.deterministic_inputs(16, 16, 16, 1, "nope")


def test_optimize_winners(golden_gemmini):
    for o in golden_gemmini["optimize"]:
        rep = g.optimize(32, 32, 32, **o["kwargs"])
        assert rep["winner"] == o["winner"]
        for got, want in zip(rep["candidates"], o["candidates"]):
            assert got["plan"]["schedule"] == want["schedule"] and got["valid"] == want["valid"]
            assert got["invalid_reason"] == want["invalid_reason"]
            assert (list(got["objective"]) if got["objective"] else None) == want["objective"]


def test_mutated_streams_are_refused_like_the_reference(golden_gemmini):
    """Mutation cases of the reference's tests/test_gemmini.py:164-206 and more; the refusal text is
    the reference interpreter's.  Every one of them is caught by the replay, before the GPU."""
    for mcase in golden_gemmini["mutations"]:
        plan = g.make_plan(32, 32, 32, mcase["schedule"])
        cmds = g.gen_commands(plan)
        name = mcase["mutation"]
        if name == "first_compute_accumulated":
            next(c for c in cmds if c.kind == "compute").accumulated = True
        elif name == "drop_all_mvout":
            cmds = [c for c in cmds if c.kind != "mvout"]
        elif name == "drop_first_mvout":
            first = next(i for i, c in enumerate(cmds) if c.kind == "mvout")
            cmds = cmds[:first] + cmds[first + 1:]
        elif name == "drop_fence":
            cmds = [c for c in cmds if c.kind != "fence"]
        elif name == "never_overwrite":
            for c in cmds:
                if c.kind == "preload":
                    c.out_addr |= g.ACCUMULATE_BIT
        elif name == "drop_config_st":
            cmds = [c for c in cmds if c.kind != "config_st"]
        elif name == "never_accumulate":
            for c in cmds:
                if c.kind == "preload":
                    c.out_addr &= ~g.ACCUMULATE_BIT
        A, B = g.deterministic_inputs(32, 32, 32, 1)
        if mcase["error"] is None:
            continue  # runs to completion in the reference: covered by the GPU tests
        with pytest.raises(g.GemminiError) as info:
            g.run_commands(cmds, plan, A, B)
        assert str(info.value) == mcase["error"], name


def test_input_validation():
    A, B = g.deterministic_inputs(16, 16, 16, 1)
    plan = g.make_plan(16, 16, 16, g.SCHEDULE_BASELINE)
    cmds = g.gen_commands(plan)
    for bad in (0.5, True, 128, -129):
        with pytest.raises(g.GemminiError):
            g.run_commands(cmds, plan, [bad] + A[1:], B)
    with pytest.raises(g.GemminiError):
        g.run_commands(cmds, plan, A[:-1], B)
    base = g.make_plan(16, 16, 16, g.SCHEDULE_BASELINE)
    for key in ("m", "k", "scratchpad_rows"):
        for bad in (16.0, True):
            p = dict(base)
            p[key] = bad
            assert g.validate_plan(p)[0] is False
    big = g.make_plan(1 << 31, 16, 16, g.SCHEDULE_BASELINE)
    ok, reason = g.validate_plan(big)
    assert not ok and "indexing" in reason


def test_fail_closed_gate():
    plan = g.make_plan(16, 16, 16, g.SCHEDULE_BASELINE)
    A, B = g.deterministic_inputs(16, 16, 16, 1)
    with mock.patch.object(g, "checker_binary_path", return_value=BIN_MISSING):
        with pytest.raises(g.GemminiError):
            g.run_commands(g.gen_commands(plan), plan, A, B)
        with pytest.raises(g.GemminiError):
            g.run_plan(plan, A, B)
        report = g.optimize(16, 16, 16)
        assert report["winner"] is None and len(report["candidates"]) == 2
        assert not any(c["check"]["accepted"] for c in report["candidates"])
    with mock.patch.object(g, "gemmini_check", return_value=(False, "mocked rejection", None)):
        with pytest.raises(g.GemminiError) as info:
            g.run_commands(g.gen_commands(plan), plan, A, B)
        assert "mocked rejection" in str(info.value)
    ok, reason, echoed = g.gemmini_check(plan)
    assert ok and echoed == plan


def test_recorded_programs_replay_to_plain_gemm(golden_gemmini):
    """The 5 accepted blind-search programs and the 8 Spike-executed streams are full GEMMs."""
    for run in golden_gemmini["recorded_hashes"] + golden_gemmini["spike_outputs"]:
        p = run["plan"]
        replay = g._Replay(p)
        for c in commands_from_dicts(run["commands"]):
            replay.step(c)
        replay.finish()
        assert g._plain_gemm_raster(replay.tiles, p["m"], p["n"], p["k"]) is not None
        if "cases" in run:
            assert replay.stats == run["cases"][0]["stats"]


def test_learned_strategy_streams_replay_like_the_reference(golden_learned_streams):
    """Streams printed by the reference's learned-strategy generators (batched A reuse, resident A, row
    batches over a resident A, serpentine B cache: scratchpad rows change roles between A and B tiles) go
    through the symbolic replay with the reference's counts and stats, or its refusal."""
    for case in golden_learned_streams["cases"]:
        plan = case["plan"]
        cmds = commands_from_dicts(case["commands"])
        assert lowering.command_hash(cmds) == case["command_sha256"], case["generator"]
        assert g.modeled_counts(cmds) == case["counts"]
        replay = g._Replay(plan)
        if "error" in case["runs"][0]:
            with pytest.raises(g.GemminiError) as info:
                for c in cmds:
                    replay.step(c)
                replay.finish()
            assert str(info.value) == case["runs"][0]["error"]
            continue
        for c in cmds:
            replay.step(c)
        replay.finish()
        assert replay.stats == case["runs"][0]["stats"], case["generator"]
        # every output tile gets each K tile of its row of A and column of B exactly once
        it, jt, kt = plan["m"] // 16, plan["n"] // 16, plan["k"] // 16
        assert len(replay.tiles) == it * jt


def test_batched_generator_argument_checks():
    plan = g.make_plan(32, 32, 32, "baseline")
    for bad in (0, -1, 1.0, True, None):
        with pytest.raises(ValueError):
            lowering.gen_batched_reuse_b(plan, bad)
    bad_plan = dict(plan, k=33)
    with pytest.raises(ValueError):
        lowering.gen_batched_reuse_b(bad_plan, 1)


def _strided_stream(stride_a, stride_b):
    """The baseline stream of a 32 x 32 x 16 plan with the load strides of A and B replaced and every mvin
    moved to the start of its buffer (or one tile along, for B's second column block), so that strides of 0, 1
    and more than a row all stay inside the buffers.  Not a GEMM any more: it runs as a tile program."""
    plan = g.make_plan(32, 32, 16, "baseline")
    cmds = g.gen_commands(plan)
    for c in cmds:
        if c.kind == "config_ld" and c.slot == 0:
            c.stride_bytes = stride_a
        elif c.kind == "config_ld" and c.slot == 1:
            c.stride_bytes = stride_b
        elif c.kind == "mvin" and c.buf == "A":
            c.offset = 0
        elif c.kind == "mvin" and c.buf == "B":
            c.offset = 16 if c.offset % 32 else 0
    return plan, cmds


def _numpy_tile_program(A, a_elems, B, b_elems, C, c_elems, lda, ldb, ldc, c_off, term_begin, a_off, b_off, **kw):
    """What vt_i8_tile_program computes, stated in numpy: tile t = sum of A-tile x B-tile products, each tile
    16 rows `stride` apart."""
    import numpy as np
    A, B = np.asarray(A, dtype=np.int64), np.asarray(B, dtype=np.int64)
    rows = np.arange(16)[:, None]
    cols = np.arange(16)[None, :]
    for t, off in enumerate(c_off):
        acc = np.zeros((16, 16), dtype=np.int64)
        for j in range(term_begin[t], term_begin[t + 1]):
            acc += A[a_off[j] + rows * lda + cols] @ B[b_off[j] + rows * ldb + cols]
        C[off + rows * ldc + cols] = acc.astype(np.int32)


@pytest.mark.parametrize("stride_a,stride_b", [(0, 32), (1, 32), (16, 0), (16, 1), (33, 32), (16, 31), (0, 0)])
def test_load_strides_reach_the_tile_program_unchanged(stride_a, stride_b):
    """config_ld strides of 0 (one row repeated), 1 (overlapping rows) and more than a row are legal in the
    reference's interpreter (specializations/gemmini_gemm/backend.py:455-459, stride_bytes >= 0); the replay must
    hand exactly those strides to the tile executor.  The executor is replaced by its numpy statement here."""
    import numpy as np
    import gemmini_oracle as go
    plan, cmds = _strided_stream(stride_a, stride_b)
    A, B = g.deterministic_inputs(32, 32, 16, 9)
    want, want_stats = go.interpret(cmds, plan, A, B)
    seen = {}

    def fake(*args, **kw):
        seen["lda"], seen["ldb"] = args[6], args[7]
        return _numpy_tile_program(*args, **kw)

    with mock.patch("veritac_b200._native.i8_tile_program", side_effect=fake):
        got, stats = g.run_commands(cmds, plan, A, B)
    assert (seen["lda"], seen["ldb"]) == (stride_a, stride_b)
    assert got == want and stats == want_stats
