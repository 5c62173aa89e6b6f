"""Tactic-by-tactic scheduling of the matmul nest with the verifier in the loop, run on the B200 back end.

The reference's examples/llm_gemm_demo.py lets a proposer (an LLM, or with --mock a fixed list) name one tactic per
step; the Lean CLI verifies and applies it to the current nest (`veritac --json`, reference Main.lean:697-745,
Search/interface.py:16-46); a rejected tactic leaves the nest unchanged and the proposer moves on; when the proposer
says "done" the final nest is timed against the untouched one through `benchmark_matmul`
(examples/llm_gemm_demo.py:260-333, 375-398).  This module is that loop for the mock proposer — the network client
belongs to the reference's Search layer and is not rebuilt — with `benchmark_matmul` being this package's: every
nest the verifier hands back is first *proved* to be the GEMM (recognise.py), then run by the CUDA kernels, and the
tile extents the schedule chose are shown beside the kernel the library picked for the shape.

The verifier is the reference's executable and nothing else: its path comes from --veritac-bin, else the
environment variable VERITAC_BIN, else `.lake/build/bin/veritac` under the current directory (where `lake build
veritac` puts it in a reference checkout).  Without it the demo stops, as the reference's does.

    VERITAC_BIN=/path/to/veritac python -m veritac_b200.examples.llm_gemm_demo --mock [--dim 256] [--runs 3]
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
from pathlib import Path

from ..specializations.cpu_gemm.runner import benchmark_matmul
from .gemm_demo import naive_matmul_stmt


def veritac_binary(explicit=None) -> Path:
    return Path(explicit or os.environ.get("VERITAC_BIN") or Path.cwd() / ".lake" / "build" / "bin" / "veritac")


def call_lean(stmt, tactics, binary=None) -> dict:
    """One round trip to the verifier: {"stmt", "applied"} or {"error"} (the contract of the reference's
    Search/interface.py:16-46).  FileNotFoundError when the executable is missing."""
    path = veritac_binary(binary)
    if not path.exists():
        raise FileNotFoundError("VeriTac binary not found at %s. Run 'lake build' first." % path)
    done = subprocess.run([str(path), "--json", json.dumps({"stmt": stmt, "tactics": tactics})], capture_output=True,
                          text=True, timeout=30)
    if done.returncode != 0:
        return {"error": "Process failed: " + done.stderr}
    try:
        return json.loads(done.stdout.strip())
    except ValueError as exc:
        return {"error": "Invalid JSON output: %s" % exc}


def _tactic(kind, *loop_vars, size=None):
    return {"kind": kind, "vars": list(loop_vars), "int_params": [] if size is None else [size], "str_params": []}


def mock_schedule(tile=32):
    """The fixed proposal list of the reference's --mock mode (examples/llm_gemm_demo.py:187-195): tile both output
    axes, bring the reduction loop above the inner column loop, vectorise that loop, parallelise the outermost."""
    return [_tactic("tile", "i0", size=tile), _tactic("tile", "i1", size=tile), _tactic("reorder", "i1_inner", "i2"),
            _tactic("vectorize", "i1_inner"), _tactic("parallel", "i0_outer")]


class MockProposer:
    """Walks a fixed list.  A proposal the verifier refused is not offered again; the walk goes on with the next
    one, and ends with "done"."""

    def __init__(self, proposals):
        self.pending = list(proposals)

    def __call__(self, schedule, stmt, last_error):
        if not self.pending:
            return {"kind": "done"}
        return self.pending.pop(0)


def describe(stmt, depth=0, out=None):
    """The nest as indented text, one loop per line."""
    out = [] if out is None else out
    pad = "  " * depth
    tag = stmt.get("tag")
    if tag == "loop":
        out.append("%sloop %s < %s  [%s]" % (pad, stmt["var"], stmt["hi"].get("val", "?"), stmt["ann"]))
        describe(stmt["body"], depth + 1, out)
    elif tag == "seq":
        describe(stmt["s1"], depth, out)
        describe(stmt["s2"], depth, out)
    elif tag == "alloc":
        out.append("%salloc %s" % (pad, stmt["buf"]))
        describe(stmt["body"], depth + 1, out)
    else:
        out.append("%s%s" % (pad, "C[..] += A[..] * B[..]" if tag == "bufWrite" else tag))
    return out


def run_agent(stmt, propose, max_steps=8, binary=None, log=print):
    """The verify-and-apply loop.  Returns (accepted tactics, final nest, [(tactic, error)] of refusals)."""
    schedule, refused, last_error = [], [], None
    for step in range(1, max_steps + 1):
        tactic = propose(schedule, stmt, last_error)
        if not tactic or tactic.get("kind") == "done":
            log("step %d: proposer is done" % step)
            break
        log("step %d: %s" % (step, json.dumps(tactic)))
        # only the new tactic goes to the verifier, applied to the current nest
        answer = call_lean(stmt, [tactic], binary)
        if "error" in answer:
            last_error = answer["error"]
            refused.append((tactic, last_error))
            log("  verifier: refused - %s (nest unchanged)" % last_error)
            continue
        last_error = None
        schedule.append(tactic)
        stmt = answer["stmt"]
        log("  verifier: applied")
        for line in describe(stmt):
            log("      " + line)
    return schedule, stmt, refused


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--dim", type=int, default=256)
    ap.add_argument("--runs", type=int, default=3)
    ap.add_argument("--max-steps", type=int, default=8)
    ap.add_argument("--mock", action="store_true", help="fixed proposal list (the only proposer built here)")
    ap.add_argument("--veritac-bin", help="path of the reference's Lean CLI (default: $VERITAC_BIN)")
    args = ap.parse_args(argv)
    if not args.mock:
        ap.error("only --mock is built here: the LLM client is part of the reference's Search layer")
    dim = args.dim
    base = naive_matmul_stmt(dim, dim, dim)
    print("== baseline nest ==")
    b0 = benchmark_matmul(base, dim, dim, dim, num_runs=args.runs)
    print("  GPU time %.4f ms   correct: %s" % (b0["c_time_ms"], b0["correct"]))
    print("== agent (mock proposer, every tactic verified before it is applied) ==")
    schedule, final, refused = run_agent(base, MockProposer(mock_schedule()), args.max_steps, args.veritac_bin)
    if not schedule:
        print("no tactic was applied; nothing to time")
        return 1
    print("== final nest ==")
    b1 = benchmark_matmul(final, dim, dim, dim, num_runs=args.runs, time_hint=True)
    print("  GPU time %.4f ms   correct: %s   relative Frobenius error vs float64: %.2e"
          % (b1["c_time_ms"], b1["correct"], b1["rel_frobenius_error"]))
    print("  numpy reference (OpenBLAS, multithreaded): %.3f ms" % b1["numpy_time_ms"])
    hint = b1["schedule_hint"]
    print("  schedule: tiles %s x %s, parallel %s, vectorize %s" % (hint["tile_m"], hint["tile_n"], hint["parallel"],
                                                                   hint["vectorize"]))
    print("  kernel the library chose for %dx%dx%d: %s (%.4f ms); kernel the schedule's tiles point at: %s (%s)"
          % (dim, dim, dim, b1["kernel"], b1["c_time_ms"], b1["hint_kernel"],
             "%.4f ms" % b1["hint_time_ms"] if b1["hint_time_ms"] is not None else "not timed"))
    print("  final schedule:")
    for t in schedule:
        print("    %s %s%s" % (t["kind"], t["vars"], t["int_params"] or ""))
    for t, why in refused:
        print("    refused: %s (%s)" % (json.dumps(t), why))
    return 0 if b0["correct"] and b1["correct"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
