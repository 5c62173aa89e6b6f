"""Parameterised Gemmini lowerings beyond the two plan schedules.

Drop-in for the generator half of the reference's specializations/gemmini_gemm/lowering.py:
`gen_batched_reuse_b` (:18-40, Lean twin VeriTac/Gemmini/Lowering.lean:26-42) and `command_hash`
(:43-45).  The certificate / rewrite-proof emission in the rest of that file belongs to the Lean
side and stays with the reference.
"""
from __future__ import annotations

import hashlib
import json

from . import backend as g

_OVERWRITE = 0xA0000000   # accumulator space | full width, overwrite
_ACCUMULATE = 0xE0000000  # accumulator space | full width | accumulate


def gen_batched_reuse_b(plan, batch_rows):
    """B-reuse with a bounded accumulator: for each column tile, `batch_rows` row tiles at a time
    stay live; each B tile is moved in once per (column, row batch, k) and latched across the batch.

    ValueError for an invalid plan or a non-positive / non-int batch size.
    """
    ok, why = g.validate_plan(plan)
    if not ok:
        raise ValueError(why)
    if type(batch_rows) is not int or batch_rows <= 0:
        raise ValueError("batch_rows must be a positive number of 16-row tiles")
    m, n, k = plan["m"], plan["n"], plan["k"]
    it, jt, kt = m // 16, n // 16, k // 16
    out = g._config_preamble(plan)
    for j in range(jt):
        for first in range(0, it, batch_rows):
            live = min(batch_rows, it - first)
            for kk in range(kt):
                out.append(g.Mvin(1, "B", (kk * n + j) * 16, 16, 16, 16))
                for local in range(live):
                    i = first + local
                    out.append(g.Mvin(0, "A", (i * k + kk) * 16, 0, 16, 16))
                    out.append(g.Preload(g.GARBAGE_ADDR if local else 16,
                                         (_ACCUMULATE if kk else _OVERWRITE) + local * 16))
                    out.append(g.Compute(local != 0, 0, g.GARBAGE_ADDR))
                    if kk == kt - 1:
                        out.append(g.Mvout((i * n + j) * 16, _ACCUMULATE + local * 16, 16, 16))
    out.append(g.Fence())
    return out


def command_hash(commands):
    """sha256 of the canonical JSON of a command list."""
    text = json.dumps(g.serialize_commands(commands), sort_keys=True, separators=(",", ":"))
    return hashlib.sha256(text.encode()).hexdigest()
