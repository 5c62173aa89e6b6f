"""Loop-nest JSON -> Python AST for the cpu_gemm path.

Drop-in for the reference's specializations/cpu_gemm/lower.py (node types :10-66, parse_expr :69-82, parse_stmt
:85-113).  Callers pattern-match on the node classes, so their names, field names and field order are the
reference's (`CLit(val)`, `CVar(name)`, `CBinOp(op, left, right)`, `CBufRead(buf, indices)`, `CSkip()`,
`CBufWrite(buf, indices, val)`, `CLoop(var, lo, hi, annotation, body)`, `CSeq(stmts)`, `CAlloc(buf, shape, body)`),
as are the JSON tags (`lit var add mul div mod bufRead` / `skip bufWrite loop seq alloc`) and the ValueError on an
unknown tag.  The JSON is what the reference's Lean CLI prints and what Search/interface.py:66-116 builds for the
naive matmul.  Here the classes are generated from one table and the two parsers are table look-ups.
"""
from __future__ import annotations

from dataclasses import dataclass, make_dataclass


@dataclass
class CExpr:
    """An integer/array expression of the loop-nest language."""


@dataclass
class CStmt:
    """A statement of the loop-nest language."""


def _node(name, base, *fields):
    cls = make_dataclass(name, list(fields), bases=(base,))
    cls.__module__ = __name__
    return cls


# expressions
CLit = _node("CLit", CExpr, ("val", int))
CVar = _node("CVar", CExpr, ("name", str))
CBinOp = _node("CBinOp", CExpr, ("op", str), ("left", CExpr), ("right", CExpr))            # op: + * / %
CBufRead = _node("CBufRead", CExpr, ("buf", str), ("indices", list))
# statements
CSkip = _node("CSkip", CStmt)
CBufWrite = _node("CBufWrite", CStmt, ("buf", str), ("indices", list), ("val", CExpr))
CLoop = _node("CLoop", CStmt, ("var", str), ("lo", CExpr), ("hi", CExpr), ("annotation", str), ("body", CStmt))
CSeq = _node("CSeq", CStmt, ("stmts", list))
CAlloc = _node("CAlloc", CStmt, ("buf", str), ("shape", list), ("body", CStmt))

_OPERATOR_OF_TAG = {"add": "+", "mul": "*", "div": "/", "mod": "%"}


def _exprs(nodes):
    return [parse_expr(n) for n in nodes]


_EXPR_BUILDERS = {
    "lit": lambda j: CLit(int(j["val"])),
    "var": lambda j: CVar(j["name"]),
    "bufRead": lambda j: CBufRead(j["buf"], _exprs(j["indices"])),
}
_STMT_BUILDERS = {
    "skip": lambda j: CSkip(),
    "bufWrite": lambda j: CBufWrite(j["buf"], _exprs(j["indices"]), parse_expr(j["val"])),
    "loop": lambda j: CLoop(j["var"], parse_expr(j["lo"]), parse_expr(j["hi"]), j.get("ann", "none"), parse_stmt(j["body"])),
    "seq": lambda j: CSeq([parse_stmt(j["s1"]), parse_stmt(j["s2"])]),
    "alloc": lambda j: CAlloc(j["buf"], _exprs(j["shape"]), parse_stmt(j["body"])),
}


def parse_expr(j: dict) -> CExpr:
    """One JSON expression node -> CExpr."""
    tag = j["tag"]
    if tag in _OPERATOR_OF_TAG:
        return CBinOp(_OPERATOR_OF_TAG[tag], parse_expr(j["left"]), parse_expr(j["right"]))
    build = _EXPR_BUILDERS.get(tag)
    if build is None:
        raise ValueError(f"Unknown expr tag: {tag}")
    return build(j)


def parse_stmt(j: dict) -> CStmt:
    """One JSON statement node -> CStmt."""
    build = _STMT_BUILDERS.get(j["tag"])
    if build is None:
        raise ValueError(f"Unknown stmt tag: {j['tag']}")
    return build(j)
