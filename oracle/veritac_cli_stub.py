#!/usr/bin/env python3
"""TEST INFRASTRUCTURE — stand-in for the reference's Lean `veritac` executable (its tactic verifier).

The reference's callers reach the verifier through one command line: `veritac --json '{"stmt": ..., "tactics":
[...]}'`, answered on stdout by one JSON object, {"stmt": ..., "applied": n} or {"error": "..."} (reference
Main.lean:697-745, processLegacy; caller side Search/interface.py:16-46).  Lean is not part of this build, so tests
point the caller's binary path here.  The tactics themselves are the restatement in loopnest_oracle.py (Tile,
Reorder, Vectorize, Parallel); anything else is answered with an error, as an unknown tactic is by the CLI.
"""
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
import loopnest_oracle as lo  # noqa: E402


def answer(text):
    try:
        req = json.loads(text)
    except ValueError as exc:
        return {"error": "JSON parse error: %s" % exc}
    if not isinstance(req, dict) or "stmt" not in req:
        return {"error": "Missing 'stmt' field"}
    tactics = req.get("tactics")
    if tactics is None:
        return {"stmt": req["stmt"]}
    try:
        out = lo.apply_tactics(req["stmt"], tactics)
    except lo.TacticError as exc:
        return {"error": str(exc)}
    except (KeyError, IndexError, TypeError) as exc:
        return {"error": "Tactic parse error: %r" % (exc,)}
    return {"stmt": out, "applied": len(tactics)}


def main(argv):
    if len(argv) == 3 and argv[1] == "--json":
        text = argv[2]
    else:
        text = sys.stdin.read().strip()
        if not text:
            print(json.dumps({"error": "No input provided. Use --json '<json>' or pipe to stdin."}))
            return 0
    print(json.dumps(answer(text), separators=(",", ":")))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
