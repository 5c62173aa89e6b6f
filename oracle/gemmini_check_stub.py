#!/usr/bin/env python3
"""TEST INFRASTRUCTURE — stand-in for the reference's Lean `gemmini_check` executable.

The reference gates every interpretation on that binary (specializations/gemmini_gemm/backend.py:
164-196) and lets its path be overridden with VERITAC_GEMMINI_CHECK_BIN (backend.py:156-159).  Lean
is not part of this build, so tests point that variable here.  The script restates the executable's
contract: plan parsing and rejection reasons of GemminiMain.lean:40-124, legality per
VeriTac/Gemmini/Plan.lean:86-92.  JSON plan on stdin (or `--json <text>`), one JSON object on
stdout: {"accepted", "reason"[, "plan"]}; the plan is echoed only on acceptance.
"""
import json
import sys

FIELDS = ("m", "n", "k", "dim", "scratchpad_rows", "accumulator_rows")


def decide(text):
    try:
        j = json.loads(text)
    except ValueError as exc:
        return {"accepted": False, "reason": "JSON parse error: %s" % exc}
    if not isinstance(j, dict):
        return {"accepted": False, "reason": "plan must be a JSON object"}
    vals = {}
    for name in FIELDS:
        v = j.get(name)
        if type(v) is not int:
            return {"accepted": False, "reason": "missing or noninteger field '%s'" % name}
        if v < 0:
            return {"accepted": False, "reason": "field '%s' must be nonnegative" % name}
        vals[name] = v
    sched = j.get("schedule")
    if not isinstance(sched, str):
        return {"accepted": False, "reason": "missing or non-string field 'schedule'"}
    if sched not in ("baseline", "reuse_b"):
        return {"accepted": False, "reason": "unknown schedule '%s'" % sched}
    m, n, k, dim = vals["m"], vals["n"], vals["k"], vals["dim"]
    ok = (m > 0 and n > 0 and k > 0 and dim > 0 and m % dim == 0 and n % dim == 0 and k % dim == 0
          and k * 16384 <= 2147483647 and vals["scratchpad_rows"] >= 2 * dim
          and vals["accumulator_rows"] >= (dim if sched == "baseline" else m))
    if not ok:
        return {"accepted": False, "reason": "plan violates planLegalProps"}
    plan = dict(vals)
    plan["schedule"] = sched
    return {"accepted": True, "reason": "accepted", "plan": plan}


def main(argv):
    text = argv[2] if len(argv) == 3 and argv[1] == "--json" else sys.stdin.read()
    text = text.strip()
    if not text:
        print(json.dumps({"accepted": False, "reason": "no input provided"}))
    else:
        print(json.dumps(decide(text), separators=(",", ":")))


if __name__ == "__main__":
    main(sys.argv)
