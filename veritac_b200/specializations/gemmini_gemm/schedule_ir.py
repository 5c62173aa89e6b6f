"""Compact schedules -> concrete command dictionaries, with resource budgets.

Counterpart of the reference's specializations/gemmini_gemm/schedule_ir.py (`expression` :30-81,
`expand_program` :84-154): a program is a list of command dictionaries and loops
`{"for": v, "start": a, "stop": b, "step": s, "body": [...]}` whose fields may be `{"expr": "..."}`
strings over integer constants and loop variables; the expansion is the flat list of dictionaries that
`run_commands` (after the strict command parser) and the byte checker see.  Same accepted language,
same refusals (`ScheduleError` with the reference's texts), same budgets.

The expression language: integer and Boolean literals, names, unary + and -, `+ - * // %`, one
comparison `== != < <= > >=`, and `x if c else y`, with Python's syntax (the text is parsed by Python's own
parser, never executed).  Text that is not a Python expression is "invalid expression"; anything Python
would accept beyond the language is refused before evaluation, wherever in the expression it stands.
"""
from __future__ import annotations

import ast
import math

_LIMIT = (1 << 64) - 1
_MAX_DEPTH = 16


class ScheduleError(ValueError):
    pass


def _bounded(value):
    if type(value) not in (int, bool) or abs(value) > _LIMIT:
        raise ScheduleError("expression value outside bounded integer domain")
    return value


# ----------------------------------------------------------------------------------------------
# Expressions.  The text is parsed by Python's own parser (so that what counts as "not an expression at
# all" is exactly what it is for the reference, indentation, comments and conditional nesting included)
# and the tree is then held to the language: a screening pass over every node, in breadth-first
# order, before anything is evaluated, and an evaluator that knows only the node kinds below.
# ----------------------------------------------------------------------------------------------
_ARITHMETIC = {
    ast.Add: lambda a, b: a + b,
    ast.Sub: lambda a, b: a - b,
    ast.Mult: lambda a, b: a * b,
    ast.FloorDiv: lambda a, b: a // b,
    ast.Mod: lambda a, b: a % b,
}
_ORDERINGS = {
    ast.Eq: lambda a, b: a == b,
    ast.NotEq: lambda a, b: a != b,
    ast.Lt: lambda a, b: a < b,
    ast.LtE: lambda a, b: a <= b,
    ast.Gt: lambda a, b: a > b,
    ast.GtE: lambda a, b: a >= b,
}
_STRUCTURE = (ast.Expression, ast.Constant, ast.Name, ast.Load, ast.UnaryOp, ast.UAdd, ast.USub, ast.BinOp,
              ast.Compare, ast.IfExp)
_IN_LANGUAGE = frozenset(_STRUCTURE) | frozenset(_ARITHMETIC) | frozenset(_ORDERINGS)


def _screen(tree, bindings):
    """Every node of the tree, used or not: its kind, its name, its literal."""
    for node in ast.walk(tree):
        kind = type(node)
        if kind not in _IN_LANGUAGE:
            raise ScheduleError("unsupported expression syntax, including in an unused branch")
        if kind is ast.Name and node.id not in bindings:
            raise ScheduleError("unbound variable")
        if kind is ast.Constant:
            _bounded(node.value)


class _Evaluator:
    def __init__(self, bindings):
        self.bindings = bindings
        self.handlers = {ast.Constant: self.constant, ast.Name: self.name, ast.UnaryOp: self.unary,
                         ast.BinOp: self.binary, ast.Compare: self.compare, ast.IfExp: self.conditional}

    def value(self, node, depth):
        if depth > _MAX_DEPTH:
            raise ScheduleError("expression nesting limit exceeded")
        handler = self.handlers.get(type(node))
        result = handler(node, depth) if handler else None
        if result is None:
            raise ScheduleError("unsupported expression or unbound variable")
        return result

    def integer_operands(self, nodes, depth, complaint):
        values = [self.value(n, depth + 1) for n in nodes]
        if any(type(v) is not int for v in values):
            raise ScheduleError(complaint)
        return values

    def constant(self, node, depth):
        return _bounded(node.value) if type(node.value) in (int, bool) else None

    def name(self, node, depth):
        return _bounded(self.bindings[node.id]) if node.id in self.bindings else None

    def unary(self, node, depth):
        if not isinstance(node.op, (ast.UAdd, ast.USub)):
            return None
        (operand,) = self.integer_operands([node.operand], depth, "arithmetic requires integers, not booleans")
        return _bounded(-operand if isinstance(node.op, ast.USub) else operand)

    def binary(self, node, depth):
        combine = _ARITHMETIC.get(type(node.op))
        if combine is None:
            return None
        left, right = self.integer_operands([node.left, node.right], depth,
                                            "arithmetic requires integers, not booleans")
        try:
            return _bounded(combine(left, right))
        except ZeroDivisionError:
            raise ScheduleError("division by zero") from None

    def compare(self, node, depth):
        if len(node.ops) != 1 or type(node.ops[0]) not in _ORDERINGS:
            return None                 # a chain a < b < c is outside the language
        left, right = self.integer_operands([node.left, node.comparators[0]], depth, "comparisons require integers")
        return _ORDERINGS[type(node.ops[0])](left, right)

    def conditional(self, node, depth):
        test = self.value(node.test, depth + 1)
        if type(test) is not bool:
            raise ScheduleError("conditional requires a Boolean test")
        return self.value(node.body if test else node.orelse, depth + 1)


def expression(source, bindings):
    """Value of `source` (int or bool) under `bindings`; ScheduleError for anything outside the language,
    unbound names and literals outside the bounded domain included, also in a branch that is not taken."""
    if not isinstance(source, str) or len(source) > 256:
        raise ScheduleError("expression must be a string of at most 256 characters")
    try:
        tree = ast.parse(source, mode="eval")
    except (SyntaxError, RecursionError):
        raise ScheduleError("invalid expression") from None
    _screen(tree, bindings)
    return _Evaluator(bindings).value(tree.body, 0)


def expand_program(program, constants, *, max_commands=4096, max_iterations=100000, max_depth=12):
    """Flat list of command dictionaries of `program`.

    A loop binds its variable (an identifier not bound already) to `range(start, stop, step)`; bounds are
    integers or `{"expr": ...}`.  Other entries are commands: a dictionary with a literal string `kind`
    whose fields are integers, Booleans, finite floats, strings or `{"expr": ...}` objects.  Budgets: at
    most `max_commands` entries per list and in the result, `max_iterations` loop iterations in total
    (counted before a loop runs, so an empty body cannot spin), `max_depth` nested lists.
    """
    for limit in (max_commands, max_iterations, max_depth):
        if type(limit) is not int or limit <= 0:
            raise ScheduleError("expansion limits must be positive integers")
    if not isinstance(constants, dict):
        raise ScheduleError("constants must be bounded named integers")
    for name, value in constants.items():
        if not isinstance(name, str) or not name.isidentifier() or type(value) is not int or abs(value) > _LIMIT:
            raise ScheduleError("constants must be bounded named integers")

    expanded = []
    spent = [0]     # loop iterations so far

    def field(value, env):
        if isinstance(value, dict):
            if set(value) != {"expr"}:
                raise ScheduleError("field object must contain only expr")
            return expression(value["expr"], env)
        if type(value) in (int, bool):
            return _bounded(value)
        if type(value) is float and math.isfinite(value) and abs(value) <= _LIMIT:
            return value
        if isinstance(value, str):
            return value
        raise ScheduleError("unsupported command field value")

    def run(entries, env, depth):
        if depth > max_depth or not isinstance(entries, list):
            raise ScheduleError("invalid program or nesting limit exceeded")
        if len(entries) > max_commands:
            raise ScheduleError("source node limit exceeded")
        for entry in entries:
            if not isinstance(entry, dict):
                raise ScheduleError("program entries must be objects")
            if "for" not in entry:
                if len(expanded) >= max_commands:
                    raise ScheduleError("expanded command budget exceeded")
                if not isinstance(entry.get("kind"), str):
                    raise ScheduleError("command needs a literal kind")
                expanded.append({key: field(value, env) for key, value in entry.items()})
                continue
            if set(entry) != {"for", "start", "stop", "step", "body"}:
                raise ScheduleError("loop fields must be for/start/stop/step/body")
            var = entry["for"]
            if not isinstance(var, str) or not var.isidentifier() or var in env:
                raise ScheduleError("loop variable invalid or shadows an existing binding")
            start, stop, step = (field(entry[key], env) for key in ("start", "stop", "step"))
            if type(start) is not int or type(stop) is not int or type(step) is not int or step == 0:
                raise ScheduleError("loop bounds require integers and nonzero step")
            values = range(start, stop, step)
            if len(values) > max_iterations - spent[0]:
                raise ScheduleError("iteration budget exceeded")
            if not isinstance(entry["body"], list):
                raise ScheduleError("loop body must be a list")
            for value in values:
                spent[0] += 1
                inner = dict(env)
                inner[var] = value
                run(entry["body"], inner, depth + 1)

    run(program, dict(constants), 0)
    return expanded
