"""TEST INFRASTRUCTURE — CPU restatement of the reference's loop-nest (cpu_gemm) semantics.

Nothing in the product imports this module.  Restated (reference paths relative to its root):
  * the naive matmul nest            Search/interface.py:66-116 (make_matmul_stmt)
  * loop-nest execution semantics    VeriTac/Schedule/LoopNest.lean:70-150 (flat index = fold of
                                     acc*1000 + idx, loops run lo..hi-1, annotations ignored); the
                                     emitted C has the same meaning (cpu_gemm/emit_c.py:29-44, 83-123)
  * the four schedule tactics        VeriTac/Tactic/Tile.lean:284-321, Reorder.lean:30-59,
                                     Vectorize.lean:23-40, Parallel.lean:23-45 — needed because the
                                     Lean CLI that applies them cannot be built here
  * the runner's operand pattern     cpu_gemm/runner.py:150-151 ((i*K+k)%7, (k*N+j)%5)
"""
from __future__ import annotations

import copy

import numpy as np

STRIDE = 1000


def lit(v):
    return {"tag": "lit", "val": int(v)}


def var(name):
    return {"tag": "var", "name": name}


def matmul_stmt(M, K, N):
    """for i0<M: for i1<N: for i2<K: C[i0,i1] = C[i0,i1] + A[i0,i2]*B[i2,i1]  (note the M,K,N order)."""
    def loop(v, hi, body):
        return {"tag": "loop", "var": v, "lo": lit(0), "hi": lit(hi), "ann": "none", "body": body}

    def rd(buf, a, b):
        return {"tag": "bufRead", "buf": buf, "indices": [var(a), var(b)]}

    write = {"tag": "bufWrite", "buf": "C", "indices": [var("i0"), var("i1")],
             "val": {"tag": "add", "left": rd("C", "i0", "i1"),
                     "right": {"tag": "mul", "left": rd("A", "i0", "i2"), "right": rd("B", "i2", "i1")}}}
    return loop("i0", M, loop("i1", N, loop("i2", K, write)))


# ------------------------------------------------------------------------------------------
# Tactics.  Each returns a new statement or raises TacticError (Lean: `none` -> CLI "error").
# ------------------------------------------------------------------------------------------
class TacticError(Exception):
    pass


def _mentions(e, name):
    t = e["tag"]
    if t == "lit":
        return False
    if t == "var":
        return e["name"] == name
    if t == "bufRead":
        return any(_mentions(i, name) for i in e["indices"])
    return _mentions(e["left"], name) or _mentions(e["right"], name)


def _static(e):
    t = e["tag"]
    if t in ("lit", "var"):
        return True
    if t == "bufRead":
        return False
    return _static(e["left"]) and _static(e["right"])


def _subst_e(e, v, rep):
    t = e["tag"]
    if t == "lit":
        return e
    if t == "var":
        return copy.deepcopy(rep) if e["name"] == v else e
    if t == "bufRead":
        return {"tag": "bufRead", "buf": e["buf"], "indices": [_subst_e(i, v, rep) for i in e["indices"]]}
    return {"tag": t, "left": _subst_e(e["left"], v, rep), "right": _subst_e(e["right"], v, rep)}


def _subst_s(s, v, rep):
    t = s["tag"]
    if t == "skip":
        return s
    if t == "bufWrite":
        return {"tag": t, "buf": s["buf"], "indices": [_subst_e(i, v, rep) for i in s["indices"]],
                "val": _subst_e(s["val"], v, rep)}
    if t == "loop":
        if s["var"] == v:
            return s
        return {"tag": t, "var": s["var"], "lo": _subst_e(s["lo"], v, rep), "hi": _subst_e(s["hi"], v, rep),
                "ann": s.get("ann", "none"), "body": _subst_s(s["body"], v, rep)}
    if t == "seq":
        return {"tag": t, "s1": _subst_s(s["s1"], v, rep), "s2": _subst_s(s["s2"], v, rep)}
    if t == "alloc":
        return {"tag": t, "buf": s["buf"], "shape": [_subst_e(i, v, rep) for i in s["shape"]],
                "body": _subst_s(s["body"], v, rep)}
    raise TacticError("unknown stmt " + t)


def _recurse(s, fn):
    """Shared traversal: first match in a loop body, else seq left then right, else alloc body."""
    t = s["tag"]
    if t == "loop":
        out = dict(s)
        out["body"] = fn(s["body"])
        return out
    if t == "seq":
        try:
            return {"tag": t, "s1": fn(s["s1"]), "s2": s["s2"]}
        except TacticError:
            return {"tag": t, "s1": s["s1"], "s2": fn(s["s2"])}
    if t == "alloc":
        out = dict(s)
        out["body"] = fn(s["body"])
        return out
    raise TacticError("target loop not found")


def tile(s, target, size):
    if s["tag"] == "loop" and s["var"] == target:
        lo, hi = s["lo"], s["hi"]
        if lo["tag"] != "lit" or hi["tag"] != "lit":
            raise TacticError("tile needs literal bounds")
        if not (size > 0 and lo["val"] == 0 and hi["val"] >= 0 and hi["val"] % size == 0):
            raise TacticError("tile size must be positive and divide the extent")
        outer, inner = target + "_outer", target + "_inner"
        rep = {"tag": "add", "left": {"tag": "mul", "left": var(outer), "right": lit(size)}, "right": var(inner)}
        return {"tag": "loop", "var": outer, "lo": lo, "hi": lit(hi["val"] // size), "ann": s.get("ann", "none"),
                "body": {"tag": "loop", "var": inner, "lo": lit(0), "hi": lit(size), "ann": "none",
                         "body": _subst_s(s["body"], target, rep)}}
    if s["tag"] in ("loop", "seq", "alloc"):
        return _recurse(s, lambda b: tile(b, target, size))
    raise TacticError("target loop not found")


def reorder(s, v1, v2):
    if s["tag"] == "loop" and s["body"]["tag"] == "loop":
        a, b = s, s["body"]
        if a["var"] == v1 and b["var"] == v2:
            safe = (not _mentions(a["lo"], v2) and not _mentions(a["hi"], v2) and _static(a["lo"])
                    and _static(a["hi"]) and not _mentions(b["lo"], v1) and not _mentions(b["hi"], v1)
                    and _static(b["lo"]) and _static(b["hi"]))
            if not safe:
                raise TacticError("loops are not swap-safe")
            inner = dict(a)
            inner["body"] = b["body"]
            out = dict(b)
            out["body"] = inner
            return out
    if s["tag"] in ("loop", "seq"):
        return _recurse(s, lambda x: reorder(x, v1, v2))
    raise TacticError("adjacent loops not found")


def _has_loop(s):
    t = s["tag"]
    if t == "loop":
        return True
    if t == "seq":
        return _has_loop(s["s1"]) or _has_loop(s["s2"])
    if t == "alloc":
        return _has_loop(s["body"])
    return False


def vectorize(s, target):
    if s["tag"] == "loop" and s["var"] == target:
        if _has_loop(s["body"]):
            raise TacticError("vectorize needs the innermost loop")
        out = dict(s)
        out["ann"] = "vectorize"
        return out
    if s["tag"] in ("loop", "seq"):
        return _recurse(s, lambda x: vectorize(x, target))
    raise TacticError("target loop not found")


def _writes(s):
    t = s["tag"]
    if t == "bufWrite":
        return [s["indices"]]
    if t == "loop" or t == "alloc":
        return _writes(s["body"])
    if t == "seq":
        return _writes(s["s1"]) + _writes(s["s2"])
    return []


def parallel(s, target):
    if s["tag"] == "loop" and s["var"] == target:
        if not all(any(_mentions(i, target) for i in idx) for idx in _writes(s["body"])):
            raise TacticError("iterations are not independent")
        out = dict(s)
        out["ann"] = "parallel"
        return out
    if s["tag"] in ("loop", "seq"):
        return _recurse(s, lambda x: parallel(x, target))
    raise TacticError("target loop not found")


def apply_tactics(stmt, tactics):
    """tactics: [{"kind", "vars", "int_params"}] in the CLI's wire form (Main.lean:697-745)."""
    for t in tactics:
        kind, vs, ps = t["kind"], t.get("vars", []), t.get("int_params", [])
        if kind == "tile":
            stmt = tile(stmt, vs[0], ps[0])
        elif kind == "reorder":
            stmt = reorder(stmt, vs[0], vs[1])
        elif kind == "vectorize":
            stmt = vectorize(stmt, vs[0])
        elif kind == "parallel":
            stmt = parallel(stmt, vs[0])
        else:
            raise TacticError("unsupported tactic " + kind)
    return stmt


# The schedule the reference's README quotes for its 256^3 number (README.md:47, :71-75).
README_SCHEDULE = [
    {"kind": "tile", "vars": ["i0"], "int_params": [32]},
    {"kind": "tile", "vars": ["i1"], "int_params": [32]},
    {"kind": "reorder", "vars": ["i1_inner", "i2"], "int_params": []},
    {"kind": "vectorize", "vars": ["i1_inner"], "int_params": []},
    {"kind": "parallel", "vars": ["i0_outer"], "int_params": []},
]


# ------------------------------------------------------------------------------------------
# Execution semantics on flat 1000-stride float64 buffers (small cases only: a Python loop).
# ------------------------------------------------------------------------------------------
def _eval(e, env, store):
    t = e["tag"]
    if t == "lit":
        return e["val"]
    if t == "var":
        return env[e["name"]]
    if t == "bufRead":
        return store[e["buf"]][_flat(e["indices"], env, store)]
    a, b = _eval(e["left"], env, store), _eval(e["right"], env, store)
    if t == "add":
        return a + b
    if t == "mul":
        return a * b
    if t == "div":
        return a // b
    if t == "mod":
        return a % b
    raise ValueError(t)


def _flat(indices, env, store):
    acc = 0
    for i in indices:
        acc = acc * STRIDE + int(_eval(i, env, store))
    return acc


def execute(stmt, store, env=None):
    env = {} if env is None else env
    t = stmt["tag"]
    if t == "skip":
        return
    if t == "bufWrite":
        store[stmt["buf"]][_flat(stmt["indices"], env, store)] = _eval(stmt["val"], env, store)
    elif t == "loop":
        for x in range(int(_eval(stmt["lo"], env, store)), int(_eval(stmt["hi"], env, store))):
            env[stmt["var"]] = x
            execute(stmt["body"], store, env)
        env.pop(stmt["var"], None)
    elif t == "seq":
        execute(stmt["s1"], store, env)
        execute(stmt["s2"], store, env)
    elif t == "alloc":
        execute(stmt["body"], store, env)
    else:
        raise ValueError(t)


def runner_operands(M, K, N, dtype=np.float64):
    """A[i,k] = (i*K+k) % 7, B[k,j] = (k*N+j) % 5 as dense row-major matrices."""
    a = (np.arange(M * K, dtype=np.int64) % 7).astype(dtype).reshape(M, K)
    b = (np.arange(K * N, dtype=np.int64) % 5).astype(dtype).reshape(K, N)
    return a, b


def runner_reference_cells(M, K, N):
    """The four cells the reference's runner compares (cpu_gemm/runner.py:216-223)."""
    a, b = runner_operands(M, K, N)
    c = a @ b
    pos = [0, STRIDE, STRIDE * (M - 1), STRIDE * (M - 1) + (N - 1)]
    return [float(c[p // STRIDE][p % STRIDE]) if p % STRIDE < N and p // STRIDE < M else float("nan") for p in pos]
