"""C/OpenMP text for a loop nest — the emitter side of the cpu_gemm path.

Drop-in for the reference's specializations/cpu_gemm/emit_c.py: emit_expr (:12-26),
flat_index_expr (:29-44), expr_mentions (:47-57), writes_local_to (:60-80), emit_stmt (:83-123),
emit_function (:126-155), emit_test_harness (:158-184).  The text is byte-identical to the
reference's for the same AST (pinned by golden fixtures), including its conventions: `double`
buffers, a fixed row stride of 1000 per index position, and an OpenMP pragma only when every write
in the loop body mentions the loop variable.  The B200 back end does not execute this text; it is
kept so callers that print, diff or compile the C keep working.
"""
from __future__ import annotations

from .lower import (CAlloc, CBinOp, CBufRead, CBufWrite, CExpr, CLit, CLoop, CSeq, CSkip, CStmt, CVar)

_INDENT = "    "


def emit_expr(e: CExpr) -> str:
    if isinstance(e, CBinOp):
        return "(%s %s %s)" % (emit_expr(e.left), e.op, emit_expr(e.right))
    if isinstance(e, CVar):
        return e.name
    if isinstance(e, CLit):
        return str(e.val)
    if isinstance(e, CBufRead):
        return "%s[%s]" % (e.buf, flat_index_expr(e.buf, e.indices))
    raise ValueError(f"Unknown CExpr type: {type(e)}")


def flat_index_expr(buf: str, indices: list[CExpr]) -> str:
    """Row-major flat index with 1000 cells per index position: i*1000^(r-1) + ... + last."""
    rank = len(indices)
    if rank == 0:
        return "0"
    terms = []
    for pos, idx in enumerate(indices):
        text = emit_expr(idx)
        if pos == rank - 1:
            terms.append(text)
        else:
            terms.append("(%s * 1%s)" % (text, " * 1000" * (rank - 1 - pos)))
    return " + ".join(terms)


def expr_mentions(e: CExpr, name: str) -> bool:
    if isinstance(e, CVar):
        return e.name == name
    if isinstance(e, CBinOp):
        return expr_mentions(e.left, name) or expr_mentions(e.right, name)
    if isinstance(e, CBufRead):
        return any(expr_mentions(i, name) for i in e.indices)
    return False


def writes_local_to(loop_var: str, stmt: CStmt) -> bool:
    """True iff every buffer write inside `stmt` has `loop_var` in its index list.

    That is when distinct iterations touch distinct cells, the condition under which a
    `parallel for` or `simd` pragma cannot change the result; a write that does not mention the
    variable is a reduction over it and gets no pragma.
    """
    if isinstance(stmt, CBufWrite):
        return any(expr_mentions(i, loop_var) for i in stmt.indices)
    if isinstance(stmt, (CLoop, CAlloc)):
        return writes_local_to(loop_var, stmt.body)
    if isinstance(stmt, CSeq):
        return all(writes_local_to(loop_var, s) for s in stmt.stmts)
    return True


def _pragma(s: CLoop, pad: str) -> str:
    if s.annotation == "parallel":
        if writes_local_to(s.var, s.body):
            return f"{pad}#pragma omp parallel for\n"
        return f"{pad}/* parallel suppressed: body writes cells not local to {s.var} */\n"
    if s.annotation == "vectorize":
        if writes_local_to(s.var, s.body):
            return f"{pad}#pragma omp simd\n"
        return f"{pad}/* simd suppressed: reduction/accumulation over {s.var} */\n"
    return ""


def emit_stmt(s: CStmt, indent: int = 1) -> str:
    pad = _INDENT * indent
    if isinstance(s, CLoop):
        head = f"{pad}for (int {s.var} = {emit_expr(s.lo)}; {s.var} < {emit_expr(s.hi)}; {s.var}++)"
        return f"{_pragma(s, pad)}{head} {{\n{emit_stmt(s.body, indent + 1)}{pad}}}\n"
    if isinstance(s, CBufWrite):
        return f"{pad}{s.buf}[{flat_index_expr(s.buf, s.indices)}] = {emit_expr(s.val)};\n"
    if isinstance(s, CSeq):
        return "".join(emit_stmt(x, indent) for x in s.stmts)
    if isinstance(s, CAlloc):
        dims = [emit_expr(d) for d in s.shape]
        return f"{pad}double {s.buf}[{' * '.join(dims) if dims else '1'}];\n" + emit_stmt(s.body, indent)
    if isinstance(s, CSkip):
        return f"{pad}/* skip */\n"
    raise ValueError(f"Unknown CStmt type: {type(s)}")


def emit_function(name: str, stmt: CStmt, input_bufs: list[tuple[str, int]],
                  output_bufs: list[tuple[str, int]]) -> str:
    """A complete translation unit: includes plus `void name(const double* in..., double* out...)`."""
    params = [f"const double* {b}" for b, _ in input_bufs] + [f"double* {b}" for b, _ in output_bufs]
    lines = ["#include <stdio.h>", "#include <stdlib.h>", "#include <string.h>", "#ifdef _OPENMP",
             "#include <omp.h>", "#endif", "", f"void {name}({', '.join(params)}) {{"]
    return "\n".join(lines) + "\n" + emit_stmt(stmt, indent=1) + "}\n"


def emit_test_harness(func_name: str, input_bufs: list[tuple[str, int]], output_bufs: list[tuple[str, int]],
                      init_code: str = "") -> str:
    """A `main` that declares the buffers, runs `init_code`, calls the function, prints 4 cells."""
    out = ["int main(void) {"]
    out += [f"    double {b}[{n}];" for b, n in input_bufs]
    for b, n in output_bufs:
        out += [f"    double {b}[{n}];", f"    memset({b}, 0, sizeof({b}));"]
    if init_code:
        out.append(init_code)
    out.append(f"    {func_name}({', '.join([b for b, _ in input_bufs] + [b for b, _ in output_bufs])});")
    for b, _ in output_bufs:
        out.append(f'    printf("{b}[0..3] = %f %f %f %f\\n", {b}[0], {b}[1], {b}[2], {b}[3]);')
    out += ["    return 0;", "}"]
    return "\n".join(out) + "\n"
