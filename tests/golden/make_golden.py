"""Regenerates tests/golden/gemmini.json, cpu_gemm.json, learned_streams.json and schedule_ir.json from the
reference tree.

Needs the reference checkout (the directory REFERENCE_ROOT names, else a directory `reference` beside this
repository) — it is imported and its
recorded evidence files are read — so it runs only where that tree exists; the fixtures it writes are
committed and are what the tests read.  The reference's Lean plan checker cannot be built here; its
documented override VERITAC_GEMMINI_CHECK_BIN (reference specializations/gemmini_gemm/backend.py:
156-159) is pointed at oracle/gemmini_check_stub.py so that the reference's *unmodified* interpreter
and generators run.

    python tests/golden/make_golden.py
"""
from __future__ import annotations

import glob
import hashlib
import json
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parents[1]
REF = Path(os.environ.get("REFERENCE_ROOT") or REPO.parent / "reference")

os.environ["VERITAC_GEMMINI_CHECK_BIN"] = str(REPO / "oracle" / "gemmini_check_stub.py")
sys.dont_write_bytecode = True
sys.path.insert(0, str(REF))
sys.path.insert(0, str(REPO / "oracle"))

from CodeGen import gemmini as g  # noqa: E402  (the reference's module)
from CodeGen import gemmini_lowering as lowering  # noqa: E402
from CodeGen import emit_c as ref_emit  # noqa: E402
from CodeGen import lower as ref_lower  # noqa: E402
from CodeGen import runner as ref_runner  # noqa: E402
from specializations.gemmini_gemm.runtime import run_raw_spike as raw  # noqa: E402

import loopnest_oracle as lo  # noqa: E402


def sha(obj) -> str:
    return hashlib.sha256(json.dumps(obj).encode()).hexdigest()


def sha_bytes(b: bytes) -> str:
    return hashlib.sha256(b).hexdigest()


def gemmini_fixture() -> dict:
    out = {"source": "CuteCake/VeriTac reference tree; see make_golden.py"}

    # 1. Full int32 outputs recorded from upstream Gemmini Spike (24 matrices).
    spike = []
    recorded_requests = [json.load(open(f)) for f in sorted(
        glob.glob(str(REF / "benchmarks/gemmini/checked*/*/request.json"))
        + glob.glob(str(REF / "benchmarks/gemmini/ai_repair/*/accepted_edge/destination/request.json")))]
    for d in sorted(glob.glob(str(REF / "benchmarks/gemmini/results/raw_*"))):
        report = json.load(open(os.path.join(d, "report.json")))
        plan = report["plan"]
        outputs = raw.parse_cout(open(os.path.join(d, "raw_spike_outputs.txt")).read())
        sizes = report["sizes"]
        modes = []
        for idx, mode in enumerate(raw.MODES):
            a, b = raw.fill_inputs(mode, sizes["A"], sizes["B"])
            modes.append({"mode": mode, "a_sha256": sha_bytes(a), "b_sha256": sha_bytes(b), "C": outputs[idx]})
        # The executed stream: the recorded request with this plan (report.json names a path outside
        # the tree), else the plan's own generator.
        commands = next((r["commands"] for r in recorded_requests if r["plan"] == plan), None)
        if commands is None:
            commands = g.serialize_commands(g.gen_commands(plan))
        spike.append({"case": os.path.basename(d), "plan": plan, "size_a": sizes["A"], "size_b": sizes["B"],
                      "commands": commands, "modes": modes})
    out["spike_outputs"] = spike

    # 2. Recorded output hashes of accepted blind-search programs (30 hashes) with their streams.
    runs = []
    base = REF / "benchmarks/gemmini/blind_search/2026-09-17/runs"
    for f in sorted(glob.glob(str(base / "*" / "local_execution.json"))):
        run = os.path.dirname(f)
        le = json.load(open(f))
        report = json.load(open(os.path.join(run, "report.json")))
        plan = report["plan"]
        req = None
        for cand in glob.glob(os.path.join(run, "**", "request.json"), recursive=True):
            r = json.load(open(cand))
            if r.get("plan") == plan and len(r.get("commands", [])) == le["cases"][0]["stats"]["instructions"]:
                req = r
                break
        if req is None:
            raise SystemExit("no request.json matches " + run)
        runs.append({"case": os.path.basename(run), "plan": plan, "commands": req["commands"],
                     "cases": [{k: c[k] for k in ("mode", "seed", "output_sha256", "stats")} for c in le["cases"]]})
    out["recorded_hashes"] = runs

    # 3. Generators: command hashes, modeled counts, interpreter stats and output hashes.
    gens = []
    shapes = [(16, 16, 16), (32, 32, 32), (48, 32, 64), (64, 64, 64), (16, 80, 32), (80, 16, 32), (32, 48, 48),
              (16, 32, 48), (48, 16, 32)]
    for (m, n, k) in shapes:
        for schedule in g.SUPPORTED_SCHEDULES:
            plan = g.make_plan(m, n, k, schedule)
            cmds = g.gen_commands(plan)
            entry = {"plan": plan, "batch_rows": None, "command_sha256": lowering.command_hash(cmds),
                     "counts": g.modeled_counts(cmds), "runs": []}
            for mode, seed in (("lcg", 1), ("lcg", 917), ("max", 0), ("min", 0), ("minmax", 0), ("zero", 0)):
                A, B = g.deterministic_inputs(m, n, k, seed, mode)
                C, stats = g.run_commands(cmds, plan, A, B)
                assert C == g.scalar_matmul(A, B, m, n, k)
                entry["runs"].append({"mode": mode, "seed": seed, "stats": stats, "output_sha256": sha(C),
                                      "a_sha256": sha(A), "b_sha256": sha(B)})
            gens.append(entry)
    for (m, n, k), acc, batches in (((48, 16, 32), 32, (1, 2)), ((64, 64, 64), 64, (1, 2, 3, 4)),
                                    ((80, 32, 48), 48, (2, 3, 5))):
        plan = g.make_plan(m, n, k, g.SCHEDULE_BASELINE)
        plan["accumulator_rows"] = acc
        for b in batches:
            entry = {"plan": plan, "batch_rows": b}
            try:
                cmds = lowering.gen_batched_reuse_b(plan, b)
                entry["command_sha256"] = lowering.command_hash(cmds)
                entry["counts"] = g.modeled_counts(cmds)
                A, B = g.deterministic_inputs(m, n, k, 5, "lcg")
                try:
                    C, stats = g.run_commands(cmds, plan, A, B)
                    entry["runs"] = [{"mode": "lcg", "seed": 5, "stats": stats, "output_sha256": sha(C),
                                      "a_sha256": sha(A), "b_sha256": sha(B)}]
                except g.GemminiError as exc:
                    entry["error"] = str(exc)
            except ValueError as exc:
                entry["value_error"] = str(exc)
            gens.append(entry)
    out["generators"] = gens

    # 4. request.json files of checked programs equal the generators' streams.
    reqs = []
    for f in sorted(glob.glob(str(REF / "benchmarks/gemmini/checked*/*/request.json"))):
        r = json.load(open(f))
        assert r["commands"] == g.serialize_commands(g.gen_commands(r["plan"])), f
        reqs.append({"case": "/".join(f.split("/")[-3:-1]), "plan": r["plan"], "n_commands": len(r["commands"]),
                     "commands_sha256": sha(r["commands"])})
    out["checked_requests"] = reqs

    # 5. validate_plan verdicts and reasons.
    base = g.make_plan(32, 32, 32, g.SCHEDULE_REUSE_B)
    variants = [{}, {"dim": 8}, {"k": 33}, {"m": 0}, {"n": 8}, {"scratchpad_rows": 16}, {"scratchpad_rows": 16385},
                {"accumulator_rows": 1025}, {"accumulator_rows": 31}, {"schedule": "baseline", "accumulator_rows": 16},
                {"schedule": "baseline", "accumulator_rows": 15}, {"schedule": "unknown"}, {"k": 131056},
                {"k": 131072}, {"m": 16.0}, {"k": True}, {"scratchpad_rows": "32"}, {"m": 2048},
                {"m": 1 << 31, "schedule": "baseline", "accumulator_rows": 16}, {"m": 8192, "n": 8192, "k": 8192},
                {"m": 8192, "n": 8192, "k": 8192, "schedule": "baseline", "accumulator_rows": 16},
                {"m": 1024, "n": 4096, "k": 4096, "schedule": "baseline", "accumulator_rows": 16}]
    verdicts = []
    for ch in variants:
        plan = dict(base)
        plan.update(ch)
        ok, reason = g.validate_plan(plan)
        verdicts.append({"plan": plan, "ok": ok, "reason": reason})
    for bad in (None, [], "plan", 42):
        ok, reason = g.validate_plan(bad)
        verdicts.append({"plan": bad, "ok": ok, "reason": reason})
    missing = dict(base)
    del missing["k"]
    ok, reason = g.validate_plan(missing)
    verdicts.append({"plan": missing, "ok": ok, "reason": reason})
    out["validate_plan"] = verdicts

    # 6. deterministic_inputs streams.
    det = []
    for (m, n, k, seed, mode) in ((16, 16, 16, 1, "lcg"), (48, 32, 64, 42, "lcg"), (64, 64, 64, 987654321, "lcg"),
                                  (16, 80, 32, 0, "lcg"), (32, 32, 32, 0, "max"), (32, 32, 32, 0, "min"),
                                  (32, 32, 32, 0, "minmax"), (32, 32, 32, 0, "zero")):
        A, B = g.deterministic_inputs(m, n, k, seed, mode)
        det.append({"args": [m, n, k, seed, mode], "a_sha256": sha(A), "b_sha256": sha(B), "a_head": A[:8],
                    "b_head": B[:8]})
    out["deterministic_inputs"] = det

    # 7. optimize(): winners under three capacity settings.
    opt = []
    for kwargs in ({}, {"scratchpad_rows": 32, "accumulator_rows": 16}, {"scratchpad_rows": 16, "accumulator_rows": 16}):
        rep = g.optimize(32, 32, 32, **kwargs)
        opt.append({"kwargs": kwargs, "winner": rep["winner"],
                    "candidates": [{"schedule": c["plan"]["schedule"], "valid": c["valid"],
                                    "invalid_reason": c["invalid_reason"], "objective": c["objective"]}
                                   for c in rep["candidates"]]})
    out["optimize"] = opt

    # 8. Mutated streams the reference refuses, with its message.
    muts = []
    for schedule in g.SUPPORTED_SCHEDULES:
        plan = g.make_plan(32, 32, 32, schedule)
        A, B = g.deterministic_inputs(32, 32, 32, 1)

        def attempt(name, cmds):
            try:
                g.run_commands(cmds, plan, A, B)
                muts.append({"schedule": schedule, "mutation": name, "error": None})
            except g.GemminiError as exc:
                muts.append({"schedule": schedule, "mutation": name, "error": str(exc)})

        cmds = g.gen_commands(plan)
        next(c for c in cmds if c.kind == "compute").accumulated = True
        attempt("first_compute_accumulated", cmds)
        attempt("drop_all_mvout", [c for c in g.gen_commands(plan) if c.kind != "mvout"])
        cmds = g.gen_commands(plan)
        first = next(i for i, c in enumerate(cmds) if c.kind == "mvout")
        attempt("drop_first_mvout", cmds[:first] + cmds[first + 1:])
        attempt("drop_fence", [c for c in g.gen_commands(plan) if c.kind != "fence"])
        cmds = g.gen_commands(plan)
        for c in cmds:
            if c.kind == "preload":
                c.out_addr |= g.ACCUMULATE_BIT
        attempt("never_overwrite", cmds)
        attempt("drop_config_st", [c for c in g.gen_commands(plan) if c.kind != "config_st"])
        cmds = g.gen_commands(plan)
        for c in cmds:
            if c.kind == "preload":
                c.out_addr &= ~g.ACCUMULATE_BIT
        attempt("never_accumulate", cmds)
    out["mutations"] = muts
    return out


def learned_streams_fixture() -> dict:
    """Command streams printed by the reference's learned-strategy generators (specializations/gemmini_gemm/
    learned_strategies.py:19-193: batched A reuse, resident A, resident A with row batches, serpentine B
    cache) with what the reference's interpreter makes of them.  The streams are data for the executor
    tests; the generators themselves are not part of this package."""
    from specializations.gemmini_gemm import learned_strategies as ls

    cases = []

    def add(name, plan, cmds):
        m, n, k = plan["m"], plan["n"], plan["k"]
        entry = {"generator": name, "plan": plan, "commands": g.serialize_commands(cmds),
                 "command_sha256": lowering.command_hash(cmds), "counts": g.modeled_counts(cmds), "runs": []}
        for mode, seed in (("lcg", 3), ("minmax", 0), ("min", 0)):
            A, B = g.deterministic_inputs(m, n, k, seed, mode)
            try:
                C, stats = g.run_commands(cmds, plan, A, B)
                assert C == g.scalar_matmul(A, B, m, n, k)
                entry["runs"].append({"mode": mode, "seed": seed, "stats": stats, "output_sha256": sha(C)})
            except g.GemminiError as exc:
                entry["runs"].append({"mode": mode, "seed": seed, "error": str(exc)})
        cases.append(entry)

    def plan_for(m, n, k, acc, spad):
        plan = g.make_plan(m, n, k, g.SCHEDULE_BASELINE)
        plan["accumulator_rows"], plan["scratchpad_rows"] = acc, spad
        return plan

    for (m, n, k, acc, batch) in ((32, 48, 48, 48, 3), (48, 80, 32, 32, 2), (16, 80, 32, 80, 5), (32, 32, 64, 16, 2)):
        plan = plan_for(m, n, k, acc, 32)
        add("gen_batched_reuse_a(batch_columns=%d)" % batch, plan, ls.gen_batched_reuse_a(plan, batch))
    for (m, n, k) in ((32, 48, 48), (16, 80, 32), (48, 32, 64)):
        plan = plan_for(m, n, k, 16, k + 16)
        add("gen_resident_a", plan, ls.gen_resident_a(plan))
    for (m, n, k, acc, batch) in ((48, 32, 32, 32, 2), (80, 16, 32, 48, 3), (64, 48, 48, 64, 4)):
        plan = plan_for(m, n, k, acc, k + 16)
        add("gen_resident_a_batched_rows(batch_rows=%d)" % batch, plan, ls.gen_resident_a_batched_rows(plan, batch))
    for (m, n, k) in ((48, 32, 32), (32, 48, 48), (64, 64, 64), (16, 32, 48)):
        plan = plan_for(m, n, k, 16, k + 16)
        add("gen_serpentine_b_cache", plan, ls.gen_serpentine_b_cache(plan))
    # select_learned_strategy needs the reference's native program checker, which cannot be built here.
    return {"source": "CuteCake/VeriTac reference tree; see make_golden.py", "cases": cases}


def schedule_ir_fixture() -> dict:
    """What the reference's compact-schedule adapter (specializations/gemmini_gemm/schedule_ir.py) makes of
    a list of expressions and programs: values, expansions, refusal texts."""
    from specializations.gemmini_gemm import schedule_ir as ir

    env = {"i": 1, "M": 32, "N": 16, "K": 32}
    texts = ["1", "i", "i*16", "i * 16 * N", "0xA0000000 if i == 0 else 0xE0000000", "K // 16", "i > 0",
             "10 if i == 0 else 20", "M.bit_length()", "2 ** 10", "M[0]", "1 / 2", "True + 1", "1 // 0", "1 << 9",
             "0 if True else int('1')", "0 if True else missing", "", " 1", "1 ", "1 # c", "1\n+2", "(1\n+2)", "--1",
             "not True", "1 < 2 < 3", "0 if True else 1 < 2 < 3", "1 == True", "True == True", "1 if 1 else 2",
             "18446744073709551615", "18446744073709551616", "18446744073709551615 + 1", "1.0", "'a'", "(1,)", "None",
             "-5 // 2", "-5 % 3", "M % 0", "1 if i > 0 else 2 if i < 0 else 3", "1 if 1 == 1 else 1 // 0", "-True",
             "True < 2", "x := 1", "(x := 1)", "M" * 300, "-" * 20 + "1", "1" + " + 1" * 20, "017", "1_000", "0b101"]
    expressions = []
    for text in texts:
        try:
            v = ir.expression(text, env)
            expressions.append({"text": text, "value": v, "is_bool": type(v) is bool})
        except ir.ScheduleError as exc:
            expressions.append({"text": text, "error": str(exc)})

    def loop(var, stop, body, start=0, step=1):
        return {"for": var, "start": start, "stop": stop, "step": step, "body": body}

    plan = g.make_plan(32, 32, 64, g.SCHEDULE_BASELINE)
    flat = g.serialize_commands(g.gen_commands(plan))
    # the baseline stream of the plan written as i, j, k loops over one tile's four commands + its mvout
    inner = [dict(c) for c in flat[4:8]]
    inner[0]["offset"] = {"expr": "(i * 16) * K + kk * 16"}
    inner[1]["offset"] = {"expr": "(kk * 16) * N + j * 16"}
    inner[2]["out_addr"] = {"expr": "0xA0000000 if kk == 0 else 0xE0000000"}
    mvout = dict(flat[4 + 4 * (plan["k"] // 16)])
    mvout["buf_offset"] = {"expr": "(i * 16) * N + j * 16"}
    compact = flat[:4] + [loop("i", {"expr": "M // 16"}, [loop("j", {"expr": "N // 16"}, [
        loop("kk", {"expr": "K // 16"}, inner), mvout])])] + flat[-1:]
    programs = [
        {"name": "baseline_32x32x64_as_loops", "program": compact, "constants": {"M": 32, "N": 32, "K": 64}, "limits": {},
         "plan": plan},
        {"name": "scoped_variable", "program": [loop("i", {"expr": "M // 16"}, [{"kind": "mvin", "offset": {"expr": "i * 16"},
                                                                                   "buf": "A"}]),
                                                 {"kind": "x", "offset": {"expr": "i"}}], "constants": {"M": 32}, "limits": {}},
        {"name": "negative_step", "program": [loop("i", -2, [{"kind": "x", "i": {"expr": "i"}}], 5, -2)], "constants": {},
         "limits": {}},
        {"name": "empty_body_budget", "program": [loop("i", 1000000000, [])], "constants": {},
         "limits": {"max_commands": 3, "max_iterations": 10}},
        {"name": "command_budget", "program": [loop("i", 5, [{"kind": "fence"}])], "constants": {},
         "limits": {"max_commands": 3, "max_iterations": 10}},
        {"name": "shadowing", "program": [loop("i", 2, [])], "constants": {"i": 1}, "limits": {}},
        {"name": "boolean_bound", "program": [loop("i", True, [])], "constants": {}, "limits": {}},
        {"name": "zero_step", "program": [loop("i", 4, [], 0, 0)], "constants": {}, "limits": {}},
        {"name": "extra_loop_field", "program": [dict(loop("i", 2, []), note=1)], "constants": {}, "limits": {}},
        {"name": "field_object", "program": [{"kind": "x", "v": {"expr": "1", "more": 2}}], "constants": {}, "limits": {}},
        {"name": "float_and_string_fields", "program": [{"kind": "config_ld", "scale": 1.0, "buf": "A", "flag": True}],
         "constants": {}, "limits": {}},
        {"name": "no_kind", "program": [{"offset": 1}], "constants": {}, "limits": {}},
        {"name": "bad_constant", "program": [], "constants": {"M": 1.5}, "limits": {}},
        {"name": "nesting", "program": [loop("a", 1, [loop("b", 1, [loop("c", 1, [{"kind": "x"}])])])], "constants": {},
         "limits": {"max_depth": 2}},
    ]
    for p in programs:
        try:
            expanded = ir.expand_program(p["program"], p["constants"], **p["limits"])
            p["expanded_sha256"] = sha_bytes(json.dumps(expanded, sort_keys=True).encode())   # key order is not data
            p["expanded_len"] = len(expanded)
            if len(expanded) <= 8:
                p["expanded"] = expanded
        except ir.ScheduleError as exc:
            p["error"] = str(exc)
    assert programs[0]["expanded_sha256"] == sha_bytes(json.dumps(flat, sort_keys=True).encode())
    return {"source": "CuteCake/VeriTac reference tree; see make_golden.py", "bindings": env, "expressions": expressions,
            "programs": programs}


def cpu_gemm_fixture() -> dict:
    out = {"source": "CuteCake/VeriTac reference tree; see make_golden.py"}

    # 1. Emitter text for a set of nests (the text itself for small nests, else its hash).
    nests = {
        "naive_4": lo.matmul_stmt(4, 4, 4),
        "naive_256": lo.matmul_stmt(256, 256, 256),
        "readme_256": lo.apply_tactics(lo.matmul_stmt(256, 256, 256), lo.README_SCHEDULE),
        "tile_parallel_256": lo.apply_tactics(lo.matmul_stmt(256, 256, 256), [
            {"kind": "tile", "vars": ["i0"], "int_params": [32]}, {"kind": "tile", "vars": ["i1"], "int_params": [32]},
            {"kind": "parallel", "vars": ["i0_outer"], "int_params": []}]),
        "parallel_on_reduction": {"tag": "loop", "var": "i2", "lo": lo.lit(0), "hi": lo.lit(8), "ann": "parallel",
                                  "body": lo.matmul_stmt(8, 8, 8)["body"]["body"]["body"]},
        "simd_on_reduction": {"tag": "loop", "var": "i2", "lo": lo.lit(0), "hi": lo.lit(8), "ann": "vectorize",
                              "body": lo.matmul_stmt(8, 8, 8)["body"]["body"]["body"]},
        "seq_alloc_skip": {"tag": "seq", "s1": {"tag": "skip"},
                           "s2": {"tag": "alloc", "buf": "T", "shape": [lo.lit(4), lo.lit(2)],
                                  "body": lo.matmul_stmt(2, 2, 2)}},
        "div_mod_rank3": {"tag": "loop", "var": "z", "lo": lo.lit(1), "hi": lo.lit(5), "ann": "unrolled",
                          "body": {"tag": "bufWrite", "buf": "S", "indices": [lo.lit(0), lo.var("z"), lo.var("z")],
                                   "val": {"tag": "mod", "left": lo.var("z"),
                                           "right": {"tag": "div", "left": lo.lit(7), "right": lo.lit(2)}}}},
        "rank0": {"tag": "bufWrite", "buf": "S", "indices": [], "val": lo.lit(3)},
    }
    emit = {}
    for name, stmt in nests.items():
        text = ref_emit.emit_function("matmul", ref_lower.parse_stmt(stmt), [("A", 1), ("B", 2)], [("C", 3)])
        emit[name] = {"stmt": stmt, "sha256": sha_bytes(text.encode()), "text": text if len(text) < 1500 else None}
    out["emit_function"] = emit
    out["emit_test_harness"] = {
        "with_init": ref_emit.emit_test_harness("f", [("A", 4)], [("C", 5)], "    A[0] = 1;"),
        "two_each": ref_emit.emit_test_harness("f", [("A", 4), ("B", 1)], [("C", 5), ("D", 1)]),
    }

    # 2. The reference runner's deterministic results (the generated OpenMP C really runs here).
    runs = []
    for (M, K, N), sched in (((64, 64, 64), None), ((256, 256, 256), None), ((256, 256, 256), "readme"),
                             ((48, 80, 32), None), ((128, 96, 160), "readme"), ((512, 512, 512), "readme")):
        stmt = lo.matmul_stmt(M, K, N)
        if sched:
            stmt = lo.apply_tactics(stmt, lo.README_SCHEDULE)
        r = ref_runner.benchmark_matmul(stmt, M, K, N, num_runs=2)
        runs.append({"M": M, "K": K, "N": N, "schedule": sched, "correct": r["correct"],
                     "c_first_values": r["c_first_values"], "np_first_values": r["np_first_values"]})
    out["benchmark_matmul"] = runs

    # 3. The tactic restatement's own pins from the reference's tests
    #    (tests/test_matmul.py:136-155, tests/test_soundness.py:41-86).
    tiled = lo.apply_tactics(lo.matmul_stmt(256, 256, 256), nests and [
        {"kind": "tile", "vars": ["i0"], "int_params": [32]}, {"kind": "tile", "vars": ["i1"], "int_params": [32]},
        {"kind": "parallel", "vars": ["i0_outer"], "int_params": []}])
    out["tactic_pins"] = {"outer_var": tiled["var"], "outer_ann": tiled["ann"], "inner_var": tiled["body"]["var"]}
    return out


if __name__ == "__main__":
    (HERE / "gemmini.json").write_text(json.dumps(gemmini_fixture(), indent=1, sort_keys=True) + "\n")
    (HERE / "cpu_gemm.json").write_text(json.dumps(cpu_gemm_fixture(), indent=1, sort_keys=True) + "\n")
    (HERE / "learned_streams.json").write_text(json.dumps(learned_streams_fixture(), sort_keys=True) + "\n")
    (HERE / "schedule_ir.json").write_text(json.dumps(schedule_ir_fixture(), indent=1, sort_keys=True) + "\n")
    print("wrote", HERE / "gemmini.json", HERE / "cpu_gemm.json")
