"""Gemmini GEMM on the B200 back end: what the model predicts beside what the GPU measures.

The reference's demo (examples/gemmini_gemm_demo.py) searches the two schedules by *modeled* traffic and says so:
"never hardware speedup".  This demo keeps the reference's gate and search (`optimize`: Lean plan check, fail
closed; winner by modeled objective) and then puts the question the model cannot answer to the hardware.  For the
winning plan it runs, through the drop-in entry points,

  * the winner's own command stream,
  * the baseline stream,
  * the batched B-reuse lowerings that fit the plan's accumulator,

each on the reference's deterministic input patterns, compares every result bit for bit with `scalar_matmul`,
and prints modeled input bytes, modeled instruction count and measured GPU time per stream side by side.

    VERITAC_GEMMINI_CHECK_BIN=/path/to/gemmini_check python -m veritac_b200.examples.gemmini_gemm_demo --m 256 --n 256 --k 256
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from ..specializations.gemmini_gemm import backend as g
from ..specializations.gemmini_gemm import evaluation

PATTERNS = (("lcg", 0x12345678), ("lcg", 0x8C0F4CC1), ("max", 0), ("minmax", 0), ("min", 0), ("zero", 0))


def check_streams_bit_exact(plan, streams):
    """Every named stream on every input pattern against scalar_matmul; {name: [pattern, ...]} of mismatches."""
    m, n, k = plan["m"], plan["n"], plan["k"]
    wrong = {}
    for mode, seed in PATTERNS:
        a, b = g.deterministic_inputs(m, n, k, seed, mode)
        want = g.scalar_matmul(a, b, m, n, k)
        for name, commands in streams.items():
            got, _stats = g.run_commands(commands, plan, a, b)
            if got != want:
                wrong.setdefault(name, []).append(mode)
    return wrong


def run_demo(m=64, n=64, k=64, scratchpad_rows=None, accumulator_rows=1024, repeats=10):
    """Returns the report dict; report["verified"] is True when a winner exists, every stream was bit-exact on
    every pattern, and the measured controls agree with one another bit for bit."""
    scratchpad_rows = g.SCRATCHPAD_ROWS if scratchpad_rows is None else scratchpad_rows
    search = g.optimize(m, n, k, scratchpad_rows=scratchpad_rows, accumulator_rows=accumulator_rows)
    report = {"shape": [m, n, k], "search": [
        {"schedule": c["plan"]["schedule"], "accepted": bool(c["valid"] and c["check"]["accepted"]),
         "reason": c["check"]["reason"] if c["valid"] else c["invalid_reason"], "objective": c.get("objective")}
        for c in search["candidates"]], "winner": search["winner"], "verified": False}
    plan = search["winner"]
    if plan is None:
        return report
    winner_stream = g.gen_commands(plan)
    a, b = g.deterministic_inputs(m, n, k, PATTERNS[0][1])
    scored = evaluation.measure_controls(plan, winner_stream, np.array(a, dtype=np.int8), np.array(b, dtype=np.int8),
                                         repeats=repeats)
    from ..specializations.gemmini_gemm.lowering import gen_batched_reuse_b
    streams = {"winner(%s)" % plan["schedule"]: winner_stream, "baseline": g.gen_baseline(plan)}
    for batch in (1, 2, 4):
        if batch * 16 <= min(m, plan["accumulator_rows"]):
            streams["batched_b_%d" % batch] = gen_batched_reuse_b(plan, batch)
    report["mismatches"] = check_streams_bit_exact(plan, streams)
    report["rows"] = [{"stream": c["name"], "modeled_input_bytes": c["counts"]["dma_in_elems_int8"],
                       "modeled_instructions": c["counts"]["instructions"], "gpu_time_ms": c["gpu_time_ms"]}
                      for c in scored["controls"] if c["native_accepted"]]
    report["rows"].append({"stream": "winner(%s)" % plan["schedule"],
                           "modeled_input_bytes": scored["counts"]["dma_in_elems_int8"],
                           "modeled_instructions": scored["counts"]["instructions"],
                           "gpu_time_ms": scored["hardware_latency"]["candidate"]})
    report["device"] = scored["hardware_latency"]["device"]
    report["controls_bit_exact"] = scored["bit_exact"]
    report["verified"] = not report["mismatches"] and scored["bit_exact"]
    return report


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--m", type=int, default=64)
    p.add_argument("--n", type=int, default=64)
    p.add_argument("--k", type=int, default=64)
    p.add_argument("--accumulator-rows", type=int, default=1024)
    p.add_argument("--repeats", type=int, default=10)
    p.add_argument("--json", help="also write the report to this file")
    args = p.parse_args(argv)
    report = run_demo(args.m, args.n, args.k, accumulator_rows=args.accumulator_rows, repeats=args.repeats)
    for s in report["search"]:
        print("plan %-9s %s (%s) objective %s" % (s["schedule"], "accepted" if s["accepted"] else "refused", s["reason"],
                                                 s["objective"]))
    if report["winner"] is None:
        print("no plan passed the gate")
        return 1
    print("winner by modeled objective: %s; measured on %s" % (report["winner"]["schedule"], report["device"]))
    print("%-22s %20s %22s %14s" % ("stream", "modeled input bytes", "modeled instructions", "GPU time (us)"))
    for r in report["rows"]:
        print("%-22s %20d %22d %14.2f" % (r["stream"], r["modeled_input_bytes"], r["modeled_instructions"],
                                          r["gpu_time_ms"] * 1e3))
    print("bit-exact on every pattern:", not report["mismatches"], "| controls agree:", report["controls_bit_exact"])
    if args.json:
        with open(args.json, "w") as fh:
            fh.write(json.dumps(report, indent=2) + "\n")
    return 0 if report["verified"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
