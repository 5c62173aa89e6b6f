"""GEMM demo on the B200 back end, after the reference's examples/gemm_demo.py:44-71.

The reference builds the naive 256^3 nest, asks its search agent and Lean CLI for a schedule, and
times both nests through `benchmark_matmul`.  The Lean CLI is not part of this build, so the scheduled
nest is either read from `--scheduled-json` (a nest the reference's `veritac --json` printed) or
built directly in the form that the README schedule — tile i0 32, tile i1 32, reorder i1_inner i2,
vectorize i1_inner, parallel i0_outer (reference README.md:47) — gives.  Both nests are proved to be
the same GEMM and run by the same kernel: on this back end a schedule is a hint, and the demo shows
exactly that (equal results, equal time), beside the numpy time the reference also prints.

    python -m veritac_b200.examples.gemm_demo [--dim 256] [--runs 3]
"""
from __future__ import annotations

import argparse
import json

from ..specializations.cpu_gemm.runner import benchmark_matmul


def _lit(v):
    return {"tag": "lit", "val": v}


def _var(n):
    return {"tag": "var", "name": n}


def _loop(v, hi, body, ann="none"):
    return {"tag": "loop", "var": v, "lo": _lit(0), "hi": _lit(hi), "ann": ann, "body": body}


def _write(i, j, k):
    rd = lambda buf, a, b: {"tag": "bufRead", "buf": buf, "indices": [a, b]}  # noqa: E731
    return {"tag": "bufWrite", "buf": "C", "indices": [i, j],
            "val": {"tag": "add", "left": rd("C", i, j), "right": {"tag": "mul", "left": rd("A", i, k),
                                                                      "right": rd("B", k, j)}}}


def naive_matmul_stmt(M, K, N):
    """The nest of the reference's Search/interface.py:66-116 (argument order M, K, N)."""
    return _loop("i0", M, _loop("i1", N, _loop("i2", K, _write(_var("i0"), _var("i1"), _var("i2")))))


def readme_scheduled_stmt(M, K, N, tile=32):
    """The nest the README schedule produces from the naive one (M and N must be multiples of `tile`)."""
    if M % tile or N % tile:
        raise ValueError("tile size must divide M and N")
    split = lambda v: {"tag": "add", "left": {"tag": "mul", "left": _var(v + "_outer"), "right": _lit(tile)},  # noqa: E731
                       "right": _var(v + "_inner")}
    body = _write(split("i0"), split("i1"), _var("i2"))
    return _loop("i0_outer", M // tile,
                 _loop("i0_inner", tile,
                       _loop("i1_outer", N // tile,
                             _loop("i2", K, _loop("i1_inner", tile, body, ann="vectorize")))), ann="parallel")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--dim", type=int, default=256)
    ap.add_argument("--runs", type=int, default=3)
    ap.add_argument("--scheduled-json", help="file holding a scheduled nest printed by the reference's Lean CLI")
    args = ap.parse_args(argv)
    dim = args.dim
    print("== Step 1: baseline nest (no tactics) ==")
    b0 = benchmark_matmul(naive_matmul_stmt(dim, dim, dim), dim, dim, dim, num_runs=args.runs)
    print(f"  baseline   GPU time: {b0['c_time_ms']:8.4f} ms   correct: {b0['correct']}")
    print("== Step 2: scheduled nest ==")
    if args.scheduled_json:
        with open(args.scheduled_json) as fh:
            loaded = json.load(fh)
        stmt = loaded.get("stmt", loaded)
    else:
        stmt = readme_scheduled_stmt(dim, dim, dim)
    b1 = benchmark_matmul(stmt, dim, dim, dim, num_runs=args.runs)
    print(f"  scheduled  GPU time: {b1['c_time_ms']:8.4f} ms   correct: {b1['correct']}")
    print(f"  end to end with host buffers: {b1['e2e_time_ms']:.3f} ms; relative Frobenius error vs float64: "
          f"{b1['rel_frobenius_error']:.2e}")
    print(f"  numpy reference (OpenBLAS, multithreaded): {b1['numpy_time_ms']:.3f} ms/eval")
    return 0 if b0["correct"] and b1["correct"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
