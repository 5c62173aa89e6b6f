"""Recognise a GEMM inside an arbitrary scheduled loop nest.

The reference compiles whatever nest it is handed (specializations/cpu_gemm/runner.py:111-190).
The B200 back end runs one operation, C[M,N] += A[M,K] * B[K,N], so before launching it proves that
the nest *is* that operation: a perfect nest of literal-bounded loops around a single
`C[i,j] = C[i,j] + A[i,k] * B[k,j]` whose three index expressions are affine in the loop variables and
enumerate [0,M) x [0,N) x [0,K) exactly once.  This accepts the naive nest of
Search/interface.py:66-116 and anything the tile / reorder / vectorize / parallel tactics
(VeriTac/Tactic/Tile.lean:284-321 and siblings) make of it, in any loop order; everything else is
refused with a reason.  fp32 summation order differs between schedules only within the stated
tolerance, so the schedule becomes a tiling hint, not a change of result.
"""
from __future__ import annotations

from .lower import CBinOp, CBufRead, CBufWrite, CExpr, CLit, CLoop, CStmt, CVar


class NotAMatmul(ValueError):
    """The loop nest is not provably the GEMM this back end executes."""


def _affine(e: CExpr) -> tuple[dict[str, int], int]:
    """e as (coefficients per variable, constant); raises NotAMatmul if e is not affine."""
    if isinstance(e, CLit):
        return {}, e.val
    if isinstance(e, CVar):
        return {e.name: 1}, 0
    if isinstance(e, CBinOp) and e.op == "+":
        (ca, ka), (cb, kb) = _affine(e.left), _affine(e.right)
        out = dict(ca)
        for v, c in cb.items():
            out[v] = out.get(v, 0) + c
        return out, ka + kb
    if isinstance(e, CBinOp) and e.op == "*":
        (ca, ka), (cb, kb) = _affine(e.left), _affine(e.right)
        if ca and cb:
            raise NotAMatmul("index expression multiplies two loop variables")
        coeffs, scale, const = (ca, kb, ka) if ca else (cb, ka, kb)
        return {v: c * scale for v, c in coeffs.items()}, const * scale
    raise NotAMatmul("index expression is not affine (div, mod or a buffer read)")


def _covers_range(form: tuple[dict[str, int], int], extents: dict[str, int], size: int, what: str) -> None:
    """The affine form must map its variables' iteration box one-to-one onto [0, size)."""
    coeffs, const = form
    coeffs = {v: c for v, c in coeffs.items() if c != 0}
    if const != 0:
        raise NotAMatmul(f"{what} index has a constant offset")
    if not coeffs:
        raise NotAMatmul(f"{what} index does not depend on any loop")
    expect = 1
    for v, c in sorted(coeffs.items(), key=lambda vc: vc[1]):
        if c != expect:
            raise NotAMatmul(f"{what} index is not a mixed-radix enumeration of its loops")
        expect *= extents[v]
    if expect != size:
        raise NotAMatmul(f"{what} index covers {expect} values, expected {size}")


def recognise_matmul(stmt: CStmt, M: int, K: int, N: int) -> dict:
    """Returns {"loops": [(var, extent, annotation, role)], ...} or raises NotAMatmul."""
    loops = []
    extents: dict[str, int] = {}
    s = stmt
    while isinstance(s, CLoop):
        if not (isinstance(s.lo, CLit) and isinstance(s.hi, CLit) and s.lo.val == 0 and s.hi.val > 0):
            raise NotAMatmul(f"loop {s.var} does not run over a literal range [0, n)")
        if s.var in extents:
            raise NotAMatmul(f"loop variable {s.var} is bound twice")
        extents[s.var] = s.hi.val
        loops.append((s.var, s.hi.val, s.annotation))
        s = s.body
    if not isinstance(s, CBufWrite) or not loops:
        raise NotAMatmul("expected a perfect loop nest around one buffer write")
    if s.buf != "C" or len(s.indices) != 2:
        raise NotAMatmul("the write must be C[i, j]")
    val = s.val
    if not (isinstance(val, CBinOp) and val.op == "+"):
        raise NotAMatmul("the written value must be C[i,j] + A[i,k] * B[k,j]")
    old, prod = (val.left, val.right) if isinstance(val.left, CBufRead) and val.left.buf == "C" else (val.right, val.left)
    if not (isinstance(old, CBufRead) and old.buf == "C" and len(old.indices) == 2):
        raise NotAMatmul("the written value must read C[i,j]")
    if not (isinstance(prod, CBinOp) and prod.op == "*" and isinstance(prod.left, CBufRead)
            and isinstance(prod.right, CBufRead)):
        raise NotAMatmul("the written value must add a product of two buffer reads")
    ra, rb = (prod.left, prod.right) if prod.left.buf == "A" else (prod.right, prod.left)
    if ra.buf != "A" or rb.buf != "B" or len(ra.indices) != 2 or len(rb.indices) != 2:
        raise NotAMatmul("the product must be A[i,k] * B[k,j]")

    wi, wj = _affine(s.indices[0]), _affine(s.indices[1])
    if (_affine(old.indices[0]), _affine(old.indices[1])) != (wi, wj):
        raise NotAMatmul("C is read and written at different cells")
    if _affine(ra.indices[0]) != wi or _affine(rb.indices[1]) != wj:
        raise NotAMatmul("A's row / B's column index differs from C's")
    wk = _affine(ra.indices[1])
    if _affine(rb.indices[0]) != wk:
        raise NotAMatmul("A's column index differs from B's row index")

    role = {}
    for name, form in (("i", wi), ("j", wj), ("k", wk)):
        for v, c in form[0].items():
            if c == 0:
                continue
            if v not in extents:
                raise NotAMatmul(f"index uses {v}, which is not a loop variable")
            if v in role:
                raise NotAMatmul(f"loop variable {v} appears in two index roles")
            role[v] = name
    unused = [v for v in extents if v not in role]
    if unused:
        raise NotAMatmul(f"loop {unused[0]} repeats the accumulation (it is in no index)")
    _covers_range(wi, extents, M, "row")
    _covers_range(wj, extents, N, "column")
    _covers_range(wk, extents, K, "reduction")
    return {"loops": [(v, n, ann, role[v]) for v, n, ann in loops], "M": M, "N": N, "K": K}
