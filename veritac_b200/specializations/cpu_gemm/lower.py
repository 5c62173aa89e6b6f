"""Loop-nest JSON -> Python AST for the cpu_gemm path.

Drop-in for the reference's specializations/cpu_gemm/lower.py (node types :10-66, parse_expr
:69-82, parse_stmt :85-113): same class names, field names and order, same JSON tags
(`lit var add mul div mod bufRead` / `skip bufWrite loop seq alloc`), same ValueError on an
unknown tag.  The JSON is what the reference's Lean CLI prints and what
Search/interface.py:66-116 builds for the naive matmul.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class CExpr:
    """An integer/array expression of the loop-nest language."""


@dataclass
class CLit(CExpr):
    val: int


@dataclass
class CVar(CExpr):
    name: str


@dataclass
class CBinOp(CExpr):
    op: str  # one of + * / %
    left: CExpr
    right: CExpr


@dataclass
class CBufRead(CExpr):
    buf: str
    indices: list[CExpr]


@dataclass
class CStmt:
    """A statement of the loop-nest language."""


@dataclass
class CSkip(CStmt):
    pass


@dataclass
class CBufWrite(CStmt):
    buf: str
    indices: list[CExpr]
    val: CExpr


@dataclass
class CLoop(CStmt):
    var: str
    lo: CExpr
    hi: CExpr
    annotation: str  # none | parallel | vectorize | unrolled
    body: CStmt


@dataclass
class CSeq(CStmt):
    stmts: list[CStmt]


@dataclass
class CAlloc(CStmt):
    buf: str
    shape: list[CExpr]
    body: CStmt


_BINARY = {"add": "+", "mul": "*", "div": "/", "mod": "%"}


def parse_expr(j: dict) -> CExpr:
    """One JSON expression node -> CExpr."""
    tag = j["tag"]
    if tag in _BINARY:
        return CBinOp(_BINARY[tag], parse_expr(j["left"]), parse_expr(j["right"]))
    if tag == "lit":
        return CLit(int(j["val"]))
    if tag == "var":
        return CVar(j["name"])
    if tag == "bufRead":
        return CBufRead(j["buf"], [parse_expr(x) for x in j["indices"]])
    raise ValueError(f"Unknown expr tag: {tag}")


def parse_stmt(j: dict) -> CStmt:
    """One JSON statement node -> CStmt."""
    tag = j["tag"]
    if tag == "loop":
        return CLoop(j["var"], parse_expr(j["lo"]), parse_expr(j["hi"]), j.get("ann", "none"),
                     parse_stmt(j["body"]))
    if tag == "bufWrite":
        return CBufWrite(j["buf"], [parse_expr(x) for x in j["indices"]], parse_expr(j["val"]))
    if tag == "seq":
        return CSeq([parse_stmt(j["s1"]), parse_stmt(j["s2"])])
    if tag == "alloc":
        return CAlloc(j["buf"], [parse_expr(x) for x in j["shape"]], parse_stmt(j["body"]))
    if tag == "skip":
        return CSkip()
    raise ValueError(f"Unknown stmt tag: {tag}")
