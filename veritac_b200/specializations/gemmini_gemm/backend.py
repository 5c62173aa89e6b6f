"""Gemmini-semantics exact int8 x int8 -> int32 full-tile GEMM, executed on a B200.

Drop-in for the execution side of the reference's specializations/gemmini_gemm/backend.py: the
same constants (:61-89), plan schema and validation (:93-149), fail-closed Lean gate (:152-196),
command classes and schedule generators (:199-343), modeled cost model (:346-373), `run_commands`
(:433-562), `scalar_matmul` (:569-580), `deterministic_inputs` (:583-602), `make_plan` / `optimize`
(:1064-1093) — same names, argument order, return shapes, exception types and refusal texts.

What differs is where the arithmetic happens.  The reference interprets the stream in Python, one
16x16x16 tile at a time.  Here `run_commands` replays the stream *symbolically* on the host — every
addressing, ordering and configuration rule of the reference interpreter is enforced, but tiles
carry (operand, offset) provenance instead of numbers — and the resulting tile program is executed
on the GPU through the C ABI: as one tcgen05 GEMM when the stream computes a full GEMM (every
generator in this module and in lowering.py does), tile by tile otherwise.  Under the plan bound
k*16384 <= 2^31-1 no accumulator can leave int32 (VeriTac/GemminiExact.lean:62-75), so the GPU's
summation order is unobservable and results are bit-identical to the interpreter's.

Carried over as they stand in the reference, because callers and the Lean side compare against their
exact verdicts and texts: `validate_plan`, `gemmini_check`, `optimize`, the command classes with their
`to_dict` forms, and the refusal strings raised during the replay.  Everything that executes — the symbolic
replay's provenance tracking, `_tile_terms`, `_plain_gemm_raster`, `_waves`, `_execute`, `run_plan` and the
numpy paths — is this package's own.

Not carried over: the Gemmini C / RV64 byte emission and the program-certificate plumbing of the
reference (its backend.py:617-1055), which stay with the reference.
"""
from __future__ import annotations

import hashlib
import json
import os
import subprocess

# ---------------------------------------------------------------------------------------------
# Hardware constants of the modeled Gemmini (reference backend.py:61-89)
# ---------------------------------------------------------------------------------------------
DIM = 16
ADDR_LEN = 32
BANK_NUM = 4
BANK_ROWS = 4096
SCRATCHPAD_ROWS = BANK_NUM * BANK_ROWS
ACC_ROWS = 1024
ELEM_MAX = 127
ELEM_MIN = -128
ACC_ELEMENT_MAX = 2**31 - 1

GARBAGE_ADDR = (1 << ADDR_LEN) - 1
ACC_SPACE_BIT = 1 << (ADDR_LEN - 1)     # bit 31: accumulator address space
ACCUMULATE_BIT = 1 << (ADDR_LEN - 2)    # bit 30: 1 accumulate onto the rows, 0 overwrite them
FULL_C_BIT = 1 << (ADDR_LEN - 3)        # bit 29: full-width (32-bit) rows
ACC_BASE_ADDR = ACC_SPACE_BIT | ACCUMULATE_BIT | FULL_C_BIT

WEIGHT_STATIONARY = 1
OUTPUT_STATIONARY = 0
NO_ACTIVATION = 0

SCHEDULE_BASELINE = "baseline"
SCHEDULE_REUSE_B = "reuse_b"
SUPPORTED_SCHEDULES = (SCHEDULE_BASELINE, SCHEDULE_REUSE_B)

INT8_DOMAIN_CONSTRAINT = "inputs are int8 in [-128,127] and k*16384 <= 2147483647"

# Most 16x16x16 products one accumulator tile can take before int32 could overflow:
# 8191 * 16 * 128 * 128 <= 2^31 - 1 < 8192 * 16 * 128 * 128.
_MAX_TERMS_PER_TILE = 8191


# ---------------------------------------------------------------------------------------------
# Plans
# ---------------------------------------------------------------------------------------------
def required_resources(plan):
    """(scratchpad_rows, accumulator_rows) the plan's schedule minimally needs."""
    rows = plan["dim"] if plan["schedule"] == SCHEDULE_BASELINE else plan["m"]
    return (2 * plan["dim"], rows)


def validate_plan(plan):
    """(ok, reason): structure, divisibility, overflow bound and capacities of a plan dict."""
    if not isinstance(plan, dict):
        return False, "plan must be a JSON object"
    for key in ("m", "n", "k", "dim", "scratchpad_rows", "accumulator_rows"):
        value = plan.get(key)
        if key not in plan or not isinstance(value, int) or isinstance(value, bool):
            return False, "plan field %r must be an integer" % key
    schedule = plan.get("schedule")
    if schedule not in SUPPORTED_SCHEDULES:
        return False, ("unsupported schedule %r (supported: %s)" % (schedule, list(SUPPORTED_SCHEDULES)))
    m, n, k, dim = plan["m"], plan["n"], plan["k"], plan["dim"]
    if dim != DIM:
        return False, "dim must equal upstream DIM=%d (got %d)" % (DIM, dim)
    for name, val in (("m", m), ("n", n), ("k", k)):
        if val < dim:
            return False, "%s=%d must be >= dim=%d" % (name, val, dim)
        if val % dim != 0:
            return False, "%s=%d must be divisible by dim=%d" % (name, val, dim)
    if k * 16384 > ACC_ELEMENT_MAX:
        return False, ("overflow bound violated: k*16384 = %d > 2147483647 (%s)"
                       % (k * 16384, INT8_DOMAIN_CONSTRAINT))
    if max(m * n, m * k, k * n) > ACC_ELEMENT_MAX:
        return False, "buffer extent exceeds the emitted C signed-int indexing range"
    need_sp, need_acc = required_resources(plan)
    sp, acc = plan["scratchpad_rows"], plan["accumulator_rows"]
    if sp < need_sp:
        return False, ("scratchpad_rows=%d < required %d for schedule %r" % (sp, need_sp, schedule))
    if sp > SCRATCHPAD_ROWS:
        return False, "scratchpad_rows=%d > hardware capacity %d" % (sp, SCRATCHPAD_ROWS)
    if acc < need_acc:
        return False, ("accumulator_rows=%d < required %d for schedule %r" % (acc, need_acc, schedule))
    if acc > ACC_ROWS:
        return False, "accumulator_rows=%d > hardware capacity %d (ACC_ROWS)" % (acc, ACC_ROWS)
    return True, "ok"


def make_plan(m, n, k, schedule):
    plan = {"m": m, "n": n, "k": k, "dim": DIM, "schedule": schedule}
    plan["scratchpad_rows"], plan["accumulator_rows"] = required_resources(plan)
    return plan


# ---------------------------------------------------------------------------------------------
# Fail-closed Lean gate
# ---------------------------------------------------------------------------------------------
def checker_binary_path():
    override = os.environ.get("VERITAC_GEMMINI_CHECK_BIN")
    if override:
        return override
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    return os.path.join(root, ".lake", "build", "bin", "gemmini_check")


def gemmini_check(plan, timeout=30):
    """(accepted, reason, echoed plan or None) from the Lean `gemmini_check` executable.

    Any absence, crash, timeout, malformed output or mismatched echo is a rejection.
    """
    path = checker_binary_path()
    if not os.path.isfile(path) or not os.access(path, os.X_OK):
        return False, ("gemmini_check binary not found or not executable at %r "
                       "(fail-closed: Lean validation required)" % path), None
    try:
        proc = subprocess.run([path], input=json.dumps(plan), capture_output=True, text=True, timeout=timeout)
    except subprocess.TimeoutExpired:
        return False, "gemmini_check timed out after %ss (fail-closed)" % timeout, None
    except OSError as exc:
        return False, "gemmini_check failed to run: %s (fail-closed)" % exc, None
    if proc.returncode != 0:
        return False, ("gemmini_check exited %d: %s (fail-closed)"
                       % (proc.returncode, (proc.stderr or proc.stdout).strip()[:400])), None
    try:
        out = json.loads(proc.stdout)
    except ValueError:
        return False, "gemmini_check emitted non-JSON output (fail-closed)", None
    if not isinstance(out, dict) or not isinstance(out.get("accepted"), bool) \
            or not isinstance(out.get("reason"), str):
        return False, "gemmini_check output missing accepted/reason (fail-closed)", None
    if out["accepted"] and out.get("plan") != plan:
        return False, "gemmini_check accepted but echoed a different plan (fail-closed)", None
    return out["accepted"], out["reason"], out.get("plan")


# ---------------------------------------------------------------------------------------------
# Command stream (fields mirror the upstream macro arguments)
# ---------------------------------------------------------------------------------------------
class Command:
    kind = "?"


class ConfigEx(Command):
    kind = "config_ex"

    def __init__(self, dataflow):
        self.dataflow = dataflow


class ConfigLd(Command):
    kind = "config_ld"

    def __init__(self, slot, stride_bytes, scale):
        self.slot = slot
        self.stride_bytes = stride_bytes
        self.scale = scale


class ConfigSt(Command):
    kind = "config_st"

    def __init__(self, stride_bytes):
        self.stride_bytes = stride_bytes


class Mvin(Command):
    kind = "mvin"

    def __init__(self, slot, buf, offset, spad_addr, cols, rows):
        self.slot = slot
        self.buf = buf
        self.offset = offset
        self.spad_addr = spad_addr
        self.cols = cols
        self.rows = rows


class Preload(Command):
    kind = "preload"

    def __init__(self, bd_spad_addr, out_addr):
        self.bd_spad_addr = bd_spad_addr
        self.out_addr = out_addr


class Compute(Command):
    kind = "compute"

    def __init__(self, accumulated, a_spad_addr, bd_spad_addr):
        self.accumulated = accumulated
        self.a_spad_addr = a_spad_addr
        self.bd_spad_addr = bd_spad_addr


class Mvout(Command):
    kind = "mvout"

    def __init__(self, buf_offset, acc_addr, cols, rows):
        self.buf_offset = buf_offset
        self.acc_addr = acc_addr
        self.cols = cols
        self.rows = rows


class Fence(Command):
    kind = "fence"


def _config_preamble(plan):
    return [ConfigEx(WEIGHT_STATIONARY), ConfigSt(plan["n"] * 4), ConfigLd(0, plan["k"], 1.0),
            ConfigLd(1, plan["n"], 1.0)]


_OVERWRITE_BASE = ACC_BASE_ADDR & ~ACCUMULATE_BIT


def gen_baseline(plan):
    """i, j, k tile order: both operand tiles move in per (i,j,k); one output tile is live."""
    m, n, k = plan["m"], plan["n"], plan["k"]
    cmds = _config_preamble(plan)
    for i in range(m // DIM):
        for j in range(n // DIM):
            for kk in range(k // DIM):
                cmds += [Mvin(0, "A", (i * k + kk) * DIM, 0, DIM, DIM),
                         Mvin(1, "B", (kk * n + j) * DIM, DIM, DIM, DIM),
                         Preload(DIM, ACC_BASE_ADDR if kk else _OVERWRITE_BASE),
                         Compute(False, 0, GARBAGE_ADDR)]
            cmds.append(Mvout((i * n + j) * DIM, ACC_BASE_ADDR, DIM, DIM))
    cmds.append(Fence())
    return cmds


def gen_reuse_b(plan):
    """j, k, i tile order: each B tile moves in once and stays latched across the i sweep."""
    m, n, k = plan["m"], plan["n"], plan["k"]
    last_k = k // DIM - 1
    cmds = _config_preamble(plan)
    for j in range(n // DIM):
        for kk in range(k // DIM):
            cmds.append(Mvin(1, "B", (kk * n + j) * DIM, DIM, DIM, DIM))
            for i in range(m // DIM):
                row = i * DIM
                cmds += [Mvin(0, "A", (i * k + kk) * DIM, 0, DIM, DIM),
                         Preload(GARBAGE_ADDR if i else DIM, (ACC_BASE_ADDR if kk else _OVERWRITE_BASE) + row),
                         Compute(i != 0, 0, GARBAGE_ADDR)]
                if kk == last_k:
                    cmds.append(Mvout((i * n + j) * DIM, ACC_BASE_ADDR + row, DIM, DIM))
    cmds.append(Fence())
    return cmds


def gen_commands(plan):
    return gen_baseline(plan) if plan["schedule"] == SCHEDULE_BASELINE else gen_reuse_b(plan)


def serialize_commands(cmds):
    """JSON-ready dicts, the only form the reference's program checker and hashes see."""
    return [dict(c) if isinstance(c, dict) else {"kind": c.kind, **vars(c)} for c in cmds]


# ---------------------------------------------------------------------------------------------
# Modeled (analytic) counts — not measurements
# ---------------------------------------------------------------------------------------------
def modeled_counts(cmds):
    counts = {key: 0 for key in ("config_ex", "config_ld", "config_st", "mvin", "preload", "compute", "mvout",
                                 "fence")}
    extra = {"mvin_A": 0, "mvin_B": 0, "compute_preloaded": 0, "compute_accumulated": 0}
    elems_in = elems_out = 0
    for c in cmds:
        counts[c.kind] += 1
        if c.kind == "mvin":
            elems_in += c.rows * c.cols
            if c.buf in ("A", "B"):
                extra["mvin_" + c.buf] += 1
        elif c.kind == "mvout":
            elems_out += c.rows * c.cols
        elif c.kind == "compute":
            extra["compute_accumulated" if c.accumulated else "compute_preloaded"] += 1
    counts.update(extra)
    counts["dma_in_elems_int8"] = elems_in
    counts["dma_out_elems_int32"] = elems_out
    counts["dma_bytes"] = elems_in + 4 * elems_out
    counts["instructions"] = len(cmds)
    return counts


def modeled_objective(counts):
    return (counts["dma_bytes"], counts["instructions"])


# ---------------------------------------------------------------------------------------------
# Execution
# ---------------------------------------------------------------------------------------------
class GemminiError(Exception):
    pass


def _as_int8(values, expected_len, what):
    """Validated int8 numpy vector from a list of Python ints or an int8 array (zero-copy)."""
    import numpy as np

    if isinstance(values, np.ndarray):
        if values.dtype != np.int8:
            raise GemminiError("%s array must have dtype int8 (got %s)" % (what, values.dtype))
        if values.size != expected_len:
            raise GemminiError("input buffers have wrong length")
        return np.ascontiguousarray(values).reshape(-1)
    if len(values) != expected_len:
        raise GemminiError("input buffers have wrong length")
    for v in values:
        if type(v) is not int or not (ELEM_MIN <= v <= ELEM_MAX):
            raise GemminiError("int8 input out of [-128,127]: %r" % (v,))
    return np.array(values, dtype=np.int8)


class _Replay:
    """Symbolic replay of a command stream: the reference interpreter's state machine
    (its backend.py:384-562) with provenance in place of numbers."""

    def __init__(self, plan):
        self.m, self.n, self.k = plan["m"], plan["n"], plan["k"]
        self.sp_rows = plan["scratchpad_rows"]
        self.acc_rows = plan["accumulator_rows"]
        self.spad = [None] * self.sp_rows          # per row: (buf, element offset of the row)
        self.acc = [None] * self.acc_rows          # per row: tuple of (a_row_ref.., ) see _compute
        self.ld_stride = {0: None, 1: None, 2: None}
        self.st_stride = None
        self.dataflow = None
        self.pending_b = None
        self.out_addr = None
        self.latched = None                        # tuple of 16 (buf, offset) rows
        self.in_flight = 0
        self.stats = {"instructions": 0, "macs": 0, "overwrites": 0, "accumulates": 0}
        self.tiles = []                            # (c_offset, stride_elems, rows) in mvout order
        self.max_acc_base = 0                      # highest accumulator row block a compute targeted

    def _spad_tile(self, start, what):
        if not (0 <= start and start + DIM <= self.sp_rows):
            raise GemminiError("%s: scratchpad rows [%d,%d) out of range" % (what, start, start + DIM))
        rows = self.spad[start:start + DIM]
        for r, row in enumerate(rows):
            if row is None:
                raise GemminiError("%s: scratchpad row %d never moved in" % (what, start + r))
        return tuple(rows)

    def _acc_base(self, addr, what):
        if not (addr & ACC_SPACE_BIT):
            raise GemminiError("%s: address %#x is not accumulator space" % (what, addr))
        if not (addr & FULL_C_BIT):
            raise GemminiError("%s: address %#x lacks full-C (bit29) width" % (what, addr))
        base = addr & (FULL_C_BIT - 1)
        if base + DIM > self.acc_rows:
            raise GemminiError("%s: accumulator rows [%d,%d) exceed ACC_ROWS=%d"
                               % (what, base, base + DIM, self.acc_rows))
        return base

    def step(self, c):
        self.stats["instructions"] += 1
        kind = c.kind
        if kind == "mvin":
            self._mvin(c)
        elif kind == "preload":
            self.pending_b = c.bd_spad_addr
            self.out_addr = c.out_addr
        elif kind == "compute":
            self._compute(c)
        elif kind == "mvout":
            self._mvout(c)
        elif kind == "config_ex":
            if c.dataflow != WEIGHT_STATIONARY:
                raise GemminiError("subset supports WEIGHT_STATIONARY only")
            self.dataflow = c.dataflow
        elif kind == "config_ld":
            if c.slot not in (0, 1, 2):
                raise GemminiError("config_ld slot %r unsupported" % c.slot)
            if c.scale != 1.0:
                raise GemminiError("subset supports MVIN_SCALE_IDENTITY only")
            if c.stride_bytes < 0:
                raise GemminiError("config_ld stride must be >= 0")
            self.ld_stride[c.slot] = c.stride_bytes
        elif kind == "config_st":
            self.st_stride = c.stride_bytes
        elif kind == "fence":
            self.in_flight = 0
        else:
            raise GemminiError("unknown command kind %r" % kind)

    def _mvin(self, c):
        stride = self.ld_stride.get(c.slot)
        if stride is None:
            raise GemminiError("mvin slot %d used before config_ld" % c.slot)
        if c.cols != DIM or c.rows != DIM:
            raise GemminiError("subset moves full %dx%d tiles only (got %dx%d)" % (DIM, DIM, c.cols, c.rows))
        if c.buf not in ("A", "B"):
            raise GemminiError("unknown input buffer")
        size = self.m * self.k if c.buf == "A" else self.k * self.n
        if not (0 <= c.offset and c.offset + (c.rows - 1) * stride + c.cols <= size):
            raise GemminiError("mvin %s: dram range out of bounds" % c.buf)
        if not (0 <= c.spad_addr and c.spad_addr + c.rows <= self.sp_rows):
            raise GemminiError("mvin: scratchpad destination out of range")
        for r in range(DIM):
            self.spad[c.spad_addr + r] = (c.buf, c.offset + r * stride)
        self.in_flight += 1

    def _compute(self, c):
        if self.dataflow != WEIGHT_STATIONARY or self.pending_b is None or self.out_addr is None:
            raise GemminiError("compute without WS configuration and preload")
        if c.bd_spad_addr != GARBAGE_ADDR:
            raise GemminiError("supported WS compute requires garbage BD operand")
        if c.accumulated:
            if self.pending_b != GARBAGE_ADDR or self.latched is None:
                raise GemminiError("compute_accumulated requires retained B weights")
        else:
            if self.pending_b == GARBAGE_ADDR:
                raise GemminiError("compute_preloaded requires an explicit B source")
            self.latched = self._spad_tile(self.pending_b, "compute preload B")
        a_rows = self._spad_tile(c.a_spad_addr, "compute A")
        base = self._acc_base(self.out_addr, "compute output")
        overwrite = not (self.out_addr & ACCUMULATE_BIT)
        b_tile = self.latched
        self.max_acc_base = max(self.max_acc_base, base)
        for r in range(DIM):
            term = (a_rows[r], b_tile)
            if overwrite:
                self.acc[base + r] = (term,)
                self.stats["overwrites"] += 1
            else:
                old = self.acc[base + r]
                if old is None:
                    raise GemminiError("accumulation into uninitialized output")
                if len(old) >= _MAX_TERMS_PER_TILE:
                    raise GemminiError("int32 accumulator overflow at acc row %d cannot be excluded after %d "
                                       "accumulations; violates %s" % (base + r, len(old), INT8_DOMAIN_CONSTRAINT))
                self.acc[base + r] = old + (term,)
                self.stats["accumulates"] += 1
        self.stats["macs"] += DIM * DIM * DIM

    def _mvout(self, c):
        if self.st_stride is None:
            raise GemminiError("mvout before config_st")
        if c.cols != DIM or c.rows != DIM:
            raise GemminiError("subset moves full %dx%d tiles only (got %dx%d)" % (DIM, DIM, c.cols, c.rows))
        stride_elems = self.st_stride // 4
        if self.st_stride % 4 != 0 or stride_elems < self.n:
            raise GemminiError("mvout stride %d bytes invalid for int32 C rows" % self.st_stride)
        if not (0 <= c.buf_offset and c.buf_offset + (c.rows - 1) * stride_elems + c.cols <= self.m * self.n):
            raise GemminiError("mvout: dram range out of bounds")
        base = self._acc_base(c.acc_addr, "mvout source")
        rows = []
        for r in range(DIM):
            row = self.acc[base + r]
            if row is None:
                raise GemminiError("read of uninitialized accumulator")
            rows.append(row)
        self.tiles.append((c.buf_offset, stride_elems, tuple(rows)))
        if self.in_flight > 0:
            self.in_flight -= 1

    def finish(self):
        if self.in_flight != 0:
            raise GemminiError("stream ended with DMAs in flight (missing fence)")


def _tile_terms(rows):
    """Per-row provenance of one moved-out tile -> list of (a_offset, lda, b_offset, ldb) tile
    products, or None when rows disagree (rows assembled from different computes)."""
    n_terms = len(rows[0])
    if any(len(r) != n_terms for r in rows):
        return None
    terms = []
    for t in range(n_terms):
        (a_buf, a0), b_tile = rows[0][t]
        if a_buf != "A" or any(b[0] != "B" for b in b_tile):
            return None
        lda = rows[1][t][0][1] - a0
        ldb = b_tile[1][1] - b_tile[0][1]
        for r in range(DIM):
            (buf_r, a_off), b_r = rows[r][t]
            if buf_r != "A" or a_off != a0 + r * lda or b_r is not b_tile and b_r != b_tile:
                return None
            if b_tile[r][1] != b_tile[0][1] + r * ldb:
                return None
        terms.append((a0, lda, b_tile[0][1], ldb))
    return terms


def _plain_gemm_raster(tiles, m, n, k):
    """If the moved-out tiles are exactly the full GEMM (every 16x16 tile of C once, each the sum over
    all K tiles of A(i,kk)*B(kk,j) with the operands' own strides) return the raster that the mvout
    order implies; else None."""
    it, jt, kt = m // DIM, n // DIM, k // DIM
    if len(tiles) != it * jt:
        return None
    seen = set()
    order = []
    for off, stride, rows in tiles:
        if stride != n or off % DIM:
            return None
        r0, c0 = divmod(off, n)
        if r0 % DIM or c0 % DIM or (r0, c0) in seen:
            return None
        terms = _tile_terms(rows)
        if terms is None or len(terms) != kt:
            return None
        want = {((r0 * k + kk * DIM), k, (kk * DIM * n + c0), n) for kk in range(kt)}
        if set(terms) != want or len(set(terms)) != kt:
            return None
        seen.add((r0, c0))
        order.append((r0 // DIM, c0 // DIM))
    if order == sorted(order):
        return "baseline"
    if order == sorted(order, key=lambda ij: (ij[1], ij[0])):
        return "reuse_b"   # also the order of the batched lowering; the caller tells them apart
    return "batched"


def _execute(plan, A, B, tiles, raster_hint=None, batch_rows=1):
    """Run the replayed program on the GPU; returns a flat int32 numpy vector of C."""
    import numpy as np

    from ... import _native as nv

    m, n, k = plan["m"], plan["n"], plan["k"]
    C = np.empty(m * n, dtype=np.int32)
    try:
        raster = _plain_gemm_raster(tiles, m, n, k) if raster_hint is None else raster_hint
        if raster == "reuse_b" and batch_rows < m // DIM:
            raster = "batched"   # column sweeps with fewer live row tiles than the matrix has
        if raster is not None:
            code = {"baseline": nv.VT_RASTER_BASELINE, "reuse_b": nv.VT_RASTER_REUSE_B,
                    "batched": nv.VT_RASTER_BATCHED}[raster]
            nv.i8gemm(A, B, C, m, n, k, raster=code, batch_rows=max(1, min(64, batch_rows)), where=nv.VT_HOST)
            return C
        # General stream: sequential waves of non-overlapping output tiles, last writer wins.
        cover = np.zeros(m * n, dtype=bool)
        C[:] = 0
        for wave in _waves(tiles, m * n):
            c_off, begin, a_off, b_off = [], [0], [], []
            lda = ldb = ldc = None
            for off, stride, rows in wave:
                terms = _tile_terms(rows)
                if terms is None:
                    raise GemminiError("stream mixes rows of different computes in one moved-out tile; "
                                       "the B200 tile executor does not run it")
                for a0, la, b0, lb in terms:
                    if (lda not in (None, la)) or (ldb not in (None, lb)):
                        raise GemminiError("stream changes operand strides mid-program; "
                                           "the B200 tile executor does not run it")
                    lda, ldb = la, lb
                    a_off.append(a0)
                    b_off.append(b0)
                if ldc not in (None, stride):
                    raise GemminiError("stream changes the output stride mid-program; "
                                       "the B200 tile executor does not run it")
                ldc = stride
                c_off.append(off)
                begin.append(len(a_off))
                idx = off + np.arange(DIM)[:, None] * stride + np.arange(DIM)[None, :]
                cover[idx.reshape(-1)] = True
            # Load strides are whatever config_ld set: 0 repeats one row, 1..15 gives overlapping rows (the
            # reference accepts any stride_bytes >= 0, backend.py:455-459); DIM only stands in when no tile has terms.
            nv.i8_tile_program(A, A.size, B, B.size, C, C.size, DIM if lda is None else lda, DIM if ldb is None else ldb, ldc,
                               np.array(c_off, dtype=np.int64), np.array(begin, dtype=np.int64),
                               np.array(a_off or [0], dtype=np.int64), np.array(b_off or [0], dtype=np.int64),
                               where=nv.VT_HOST)
        if not cover.all():
            raise GemminiError("not every output element was written")
        return C
    except nv.NativeError as exc:
        raise GemminiError("B200 execution failed: %s" % exc) from exc


def _waves(tiles, c_elems):
    """Split mvouts into launches whose tiles do not overlap; a later mvout to the very same
    offset replaces the earlier one inside a wave."""
    waves, current, cells = [], {}, set()
    for off, stride, rows in tiles:
        own = {off + r * stride + c for r in range(DIM) for c in range(DIM)}
        if off in current and current[off][1] == stride:
            current[off] = (off, stride, rows)
            continue
        if cells & own:
            waves.append(list(current.values()))
            current, cells = {}, set()
        current[off] = (off, stride, rows)
        cells |= own
    if current:
        waves.append(list(current.values()))
    return waves


def run_commands(cmds, plan, A, B):
    """Execute a command stream under the declared subset contract; returns (C, stats).

    C is a list of m*n Python ints when A and B are lists (the reference's form) and an int32 numpy
    vector when they are int8 numpy arrays.  GemminiError on an invalid plan, a rejecting or missing
    Lean checker, malformed inputs, and every subset / addressing / ordering violation the
    reference interpreter reports.
    """
    ok, reason = validate_plan(plan)
    if not ok:
        raise GemminiError(reason)
    accepted, reason, _ = gemmini_check(plan)
    if not accepted:
        raise GemminiError("Lean rejected interpretation: " + reason)
    m, n, k = plan["m"], plan["n"], plan["k"]
    as_list = not hasattr(A, "dtype")
    a8 = _as_int8(A, m * k, "A")
    b8 = _as_int8(B, k * n, "B")
    replay = _Replay(plan)
    for c in cmds:
        replay.step(c)
    replay.finish()
    covered = set()
    for off, stride, _rows in replay.tiles:
        for r in range(DIM):
            covered.update(range(off + r * stride, off + r * stride + DIM))
    if len(covered) != m * n:
        raise GemminiError("not every output element was written")
    C = _execute(plan, a8, b8, replay.tiles, batch_rows=replay.max_acc_base // DIM + 1)
    return ([int(v) for v in C] if as_list else C), replay.stats


def run_plan(plan, A, B, batch_rows=None):
    """Execute the plan's own schedule without materialising its command list; returns (C, stats).

    For sizes where the list form is impractical (an 8192^3 baseline stream has 5.4e8 commands).
    The result and `stats` equal run_commands(gen_commands(plan), ...) — or, with `batch_rows`,
    run_commands(gen_batched_reuse_b(plan, batch_rows), ...) — computed in closed form.  A and B are
    lists of ints or int8 numpy arrays.  Same gate and refusals as run_commands.
    """
    ok, reason = validate_plan(plan)
    if not ok:
        raise GemminiError(reason)
    accepted, reason, _ = gemmini_check(plan)
    if not accepted:
        raise GemminiError("Lean rejected interpretation: " + reason)
    m, n, k = plan["m"], plan["n"], plan["k"]
    it, jt, kt = m // DIM, n // DIM, k // DIM
    if batch_rows is not None:
        if type(batch_rows) is not int or batch_rows <= 0:
            raise ValueError("batch_rows must be a positive number of 16-row tiles")
        fit = plan["accumulator_rows"] // DIM          # row blocks the accumulator can hold
        if min(batch_rows, it) > fit:                  # the stream's first compute beyond capacity
            raise GemminiError("compute output: accumulator rows [%d,%d) exceed ACC_ROWS=%d"
                               % (fit * DIM, fit * DIM + DIM, plan["accumulator_rows"]))
        raster, b_loads = "batched", jt * kt * ((it + batch_rows - 1) // batch_rows)
    elif plan["schedule"] == SCHEDULE_BASELINE:
        raster, b_loads = "baseline", it * jt * kt
    else:
        raster, b_loads = "reuse_b", jt * kt
    as_list = not hasattr(A, "dtype")
    a8 = _as_int8(A, m * k, "A")
    b8 = _as_int8(B, k * n, "B")
    computes = it * jt * kt
    stats = {"instructions": 4 + b_loads + 3 * computes + it * jt + 1, "macs": computes * DIM ** 3,
             "overwrites": it * jt * DIM, "accumulates": it * jt * (kt - 1) * DIM}
    C = _execute(plan, a8, b8, None, raster_hint=raster, batch_rows=batch_rows or 1)
    return ([int(v) for v in C] if as_list else C), stats


def scalar_matmul(A, B, m, n, k):
    """Exact C[i*n+j] = sum_t A[i*k+t] * B[t*n+j], on the GPU.

    Lists in, list out (numpy int8 in, numpy int32 out).  Any positive m, n, k: operands are
    zero-padded to multiples of 16 for the kernel.  GemminiError when an input is not an int8 value or
    k is beyond the bound under which int32 cannot overflow.
    """
    import numpy as np

    from ... import _native as nv

    if k * 16384 > ACC_ELEMENT_MAX:
        raise GemminiError("reference overflow (plan violates %s)" % INT8_DOMAIN_CONSTRAINT)
    as_list = not hasattr(A, "dtype")
    a8 = _as_int8(A, m * k, "A").reshape(m, k)
    b8 = _as_int8(B, k * n, "B").reshape(k, n)
    mp, np_, kp = (-(-m // DIM) * DIM, -(-n // DIM) * DIM, -(-k // DIM) * DIM)
    if (mp, np_, kp) != (m, n, k):
        ap = np.zeros((mp, kp), dtype=np.int8)
        bp = np.zeros((kp, np_), dtype=np.int8)
        ap[:m, :k] = a8
        bp[:k, :n] = b8
        a8, b8 = ap, bp
    C = np.empty((mp, np_), dtype=np.int32)
    try:
        nv.i8gemm(np.ascontiguousarray(a8), np.ascontiguousarray(b8), C, mp, np_, kp, where=nv.VT_HOST)
    except nv.NativeError as exc:
        raise GemminiError("B200 execution failed: %s" % exc) from exc
    C = np.ascontiguousarray(C[:m, :n]).reshape(-1)
    return [int(v) for v in C] if as_list else C


def deterministic_inputs(m, n, k, seed, mode="lcg"):
    """(A, B) as lists of ints: an LCG stream (A first, B continuing it) or a constant pattern."""
    if mode == "lcg":
        x = seed & 0xFFFFFFFF
        vals = []
        for _ in range(m * k + k * n):
            x = (1103515245 * x + 12345) & 0xFFFFFFFF
            vals.append((x >> 16) % 256 - 128)
        return vals[:m * k], vals[m * k:]
    fills = {"max": (ELEM_MAX, ELEM_MAX), "minmax": (ELEM_MIN, ELEM_MAX), "min": (ELEM_MIN, ELEM_MIN),
             "zero": (0, 0)}
    if mode not in fills:
        raise ValueError(mode)
    a, b = fills[mode]
    return [a] * (m * k), [b] * (k * n)


def sha256_file(path):
    digest = hashlib.sha256()
    with open(path, "rb") as fh:
        for chunk in iter(lambda: fh.read(65536), b""):
            digest.update(chunk)
    return digest.hexdigest()


# ---------------------------------------------------------------------------------------------
# Schedule selection by the modeled objective
# ---------------------------------------------------------------------------------------------
def optimize(m, n, k, *, scratchpad_rows=SCRATCHPAD_ROWS, accumulator_rows=ACC_ROWS):
    """Both schedules against the same capacities; winner = least modeled DMA bytes, then fewest
    instructions, then fewest required accumulator rows, among valid and Lean-accepted plans."""
    candidates = []
    for schedule in SUPPORTED_SCHEDULES:
        plan = make_plan(m, n, k, schedule)
        plan.update(scratchpad_rows=scratchpad_rows, accumulator_rows=accumulator_rows)
        ok, reason = validate_plan(plan)
        accepted, chk_reason, _ = gemmini_check(plan)
        entry = {"plan": plan, "valid": ok, "invalid_reason": None if ok else reason,
                 "check": {"accepted": accepted, "reason": chk_reason}, "counts": None, "objective": None}
        if ok and accepted:
            entry["counts"] = modeled_counts(gen_commands(plan))
            entry["objective"] = modeled_objective(entry["counts"]) + (required_resources(plan)[1],)
        candidates.append(entry)
    eligible = [c for c in candidates if c["valid"] and c["check"]["accepted"]]
    winner = min(eligible, key=lambda c: c["objective"])["plan"] if eligible else None
    return {"candidates": candidates, "winner": winner}
