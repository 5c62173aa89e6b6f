"""TEST INFRASTRUCTURE — CPU restatement of the reference's Gemmini int8 GEMM semantics.

Nothing in the product imports this module; only tests/, __graft_entry__.smoke() and the
cpu_baseline / reference legs of bench.py do, and only as the checker.

What is restated (reference = CuteCake/VeriTac, paths relative to its root):
  * scalar reference            specializations/gemmini_gemm/backend.py:569-580 (scalar_matmul)
                                and its C twin :711-720 (veritac_scalar_ref)
  * sequential interpreter      backend.py:384-562 (GemminiState, run_commands)
  * deterministic inputs        backend.py:583-602 (deterministic_inputs)
  * raw-harness input patterns  specializations/gemmini_gemm/runtime/run_raw_spike.py:133-151
  * COUT parsing                run_raw_spike.py:409-423 (parse_cout)
  * plan legality               VeriTac/Gemmini/Plan.lean:86-92 (planLegalProps)

Parity of this oracle is pinned by tests/test_oracle_golden.py against the reference's recorded
Spike outputs, output hashes, command streams and checker cases (fixtures in tests/golden/).
"""
from __future__ import annotations

import hashlib
import json
import re

import numpy as np

DIM = 16
GARBAGE = 0xFFFFFFFF
BIT_ACC = 1 << 31
BIT_ACCUMULATE = 1 << 30
BIT_FULL = 1 << 29
INT32_MAX = 2**31 - 1
INT32_MIN = -(2**31)


class OracleError(Exception):
    """The stream or its inputs violate the declared subset (reference: GemminiError)."""


# --------------------------------------------------------------------------------------------
# Exact products
# --------------------------------------------------------------------------------------------
def matmul_exact(A, B, m, n, k):
    """C[i,j] = sum_t A[i,t] * B[t,j] over the integers, as int64 (backend.py:569-580).

    Uses float64 BLAS: every product is at most 2^14 in magnitude and every partial sum at most
    k * 2^14, exact in a double while k * 2^14 < 2^53.
    """
    a = np.asarray(A, dtype=np.int64).reshape(m, k)
    b = np.asarray(B, dtype=np.int64).reshape(k, n)
    if k * 16384 >= 2**53:
        raise OracleError("k too large for the float64-exact path")
    c = a.astype(np.float64) @ b.astype(np.float64)
    return np.rint(c).astype(np.int64)


def scalar_matmul(A, B, m, n, k):
    """List-in, list-out twin of the reference scalar_matmul, including its overflow refusal."""
    c = matmul_exact(A, B, m, n, k)
    if c.size and (c.max() > INT32_MAX or c.min() < INT32_MIN):
        raise OracleError("reference overflow")
    return [int(v) for v in c.reshape(-1)]


def scalar_matmul_loops(A, B, m, n, k):
    """The literal triple loop (small cases only): pins matmul_exact itself."""
    C = [0] * (m * n)
    for i in range(m):
        for j in range(n):
            s = 0
            for t in range(k):
                s += A[i * k + t] * B[t * n + j]
            C[i * n + j] = s
    return C


# --------------------------------------------------------------------------------------------
# Inputs
# --------------------------------------------------------------------------------------------
def _lcg_states(count, seed):
    """count successive states of x <- 1103515245 x + 12345 (mod 2^32), vectorised by doubling."""
    out = np.empty(count, dtype=np.uint64)
    mask = np.uint64(0xFFFFFFFF)
    a, c = 1103515245, 12345
    x = seed & 0xFFFFFFFF
    # plain loop for short streams, jump-ahead blocks for long ones
    if count <= 4096:
        for i in range(count):
            x = (a * x + c) & 0xFFFFFFFF
            out[i] = x
        return out
    block = 4096
    first = np.empty(block, dtype=np.uint64)
    for i in range(block):
        x = (a * x + c) & 0xFFFFFFFF
        first[i] = x
    # x_{i+block} = A_b x_i + C_b
    ab, cb = 1, 0
    for _ in range(block):
        ab, cb = (ab * a) & 0xFFFFFFFF, (cb * a + c) & 0xFFFFFFFF
    ab64, cb64 = np.uint64(ab), np.uint64(cb)
    cur = first
    pos = 0
    while pos < count:
        take = min(block, count - pos)
        out[pos:pos + take] = cur[:take]
        pos += take
        cur = (cur * ab64 + cb64) & mask
    return out


def deterministic_inputs(m, n, k, seed, mode="lcg"):
    """(A, B) as int8 numpy vectors; same streams as backend.py:583-602."""
    if mode == "lcg":
        s = _lcg_states(m * k + k * n, seed)
        vals = ((s >> np.uint64(16)) % np.uint64(256)).astype(np.int64) - 128
        return vals[:m * k].astype(np.int8), vals[m * k:].astype(np.int8)
    table = {"max": (127, 127), "minmax": (-128, 127), "min": (-128, -128), "zero": (0, 0)}
    if mode not in table:
        raise ValueError(mode)
    a, b = table[mode]
    return np.full(m * k, a, dtype=np.int8), np.full(k * n, b, dtype=np.int8)


RAW_MODES = ("zeros", "extrema", "lcg")


def raw_fill_inputs(mode, size_a, size_b):
    """(A, B) as int8 vectors for the raw-Spike harness modes (run_raw_spike.py:133-151)."""
    if mode == "zeros":
        return np.zeros(size_a, dtype=np.int8), np.zeros(size_b, dtype=np.int8)
    if mode == "extrema":
        ia = np.arange(size_a)
        ib = np.arange(size_b)
        a = np.where(ia % 2 == 0, 0x80, 0x7F).astype(np.uint8).view(np.int8)
        b = np.where(ib % 2 == 0, 0x7F, 0x80).astype(np.uint8).view(np.int8)
        return a, b
    if mode == "lcg":
        s = _lcg_states(size_a + size_b, 0x12345678)
        by = ((s >> np.uint64(16)) & np.uint64(0xFF)).astype(np.uint8).view(np.int8)
        return by[:size_a].copy(), by[size_a:].copy()
    raise ValueError(mode)


_COUT = re.compile(r"^COUT (\d+) ([0-9a-f]+)$")


def parse_cout(text):
    """{mode index: int32 list} from the harness' `COUT <mode> %08x...` lines."""
    out = {}
    for line in text.splitlines():
        mt = _COUT.match(line)
        if not mt:
            continue
        payload = mt.group(2)
        if len(payload) % 8:
            raise OracleError("malformed COUT payload")
        words = np.array([int(payload[i:i + 8], 16) for i in range(0, len(payload), 8)], dtype=np.uint32)
        out[int(mt.group(1))] = words.view(np.int32).astype(np.int64).tolist()
    return out


def output_sha256(C):
    """sha256 over json.dumps(list of ints): the recipe of the reference's recorded output hashes
    (benchmarks/gemmini/blind_search/2026-09-17/check_local_execution.py:47-55)."""
    return hashlib.sha256(json.dumps([int(v) for v in C]).encode()).hexdigest()


# --------------------------------------------------------------------------------------------
# Plan legality (Lean side) — what the gemmini_check binary decides
# --------------------------------------------------------------------------------------------
def plan_legal(plan):
    """(accepted, reason) for an already well-typed plan dict, per planLegalProps."""
    m, n, k, dim = plan["m"], plan["n"], plan["k"], plan["dim"]
    sp, acc = plan["scratchpad_rows"], plan["accumulator_rows"]
    if not (m > 0 and n > 0 and k > 0 and dim > 0):
        return False, "m, n, k and dim must be positive"
    if m % dim or n % dim or k % dim:
        return False, "m, n and k must be divisible by dim"
    if k * 16384 > INT32_MAX:
        return False, "k * 16384 exceeds 2^31 - 1"
    if sp < 2 * dim:
        return False, "scratchpad_rows below 2 * dim"
    need = dim if plan["schedule"] == "baseline" else m
    if acc < need:
        return False, "accumulator_rows below the schedule's requirement"
    return True, "accepted"


# --------------------------------------------------------------------------------------------
# Sequential interpreter over command dicts (the serialize_commands form: {"kind": ..., fields})
# --------------------------------------------------------------------------------------------
def as_dicts(cmds):
    return [dict(c) if isinstance(c, dict) else {"kind": c.kind, **vars(c)} for c in cmds]


def interpret(cmds, plan, A, B):
    """Run a command stream one instruction at a time.  Returns (C list, stats)."""
    m, n, k = plan["m"], plan["n"], plan["k"]
    sp_rows, acc_rows = plan["scratchpad_rows"], plan["accumulator_rows"]
    if len(A) != m * k or len(B) != k * n:
        raise OracleError("input buffers have wrong length")
    for v in list(A) + list(B):
        if type(v) is not int or not -128 <= v <= 127:
            raise OracleError("int8 input out of range: %r" % (v,))
    src = {"A": np.array(A, dtype=np.int64), "B": np.array(B, dtype=np.int64)}
    size = {"A": m * k, "B": k * n}
    spad = [None] * sp_rows
    acc = [None] * acc_rows
    C = [0] * (m * n)
    written = [False] * (m * n)
    ld_stride = {0: None, 1: None, 2: None}
    st_stride = None
    dataflow = None
    pending_b = None
    out_addr = None
    latched = None
    in_flight = 0
    stats = {"instructions": 0, "macs": 0, "overwrites": 0, "accumulates": 0}

    def spad_tile(row, what):
        if not (0 <= row and row + DIM <= sp_rows):
            raise OracleError("%s: scratchpad rows out of range" % what)
        rows = spad[row:row + DIM]
        if any(r is None for r in rows):
            raise OracleError("%s: scratchpad row never moved in" % what)
        return np.stack(rows)

    def acc_base(addr, what):
        if not addr & BIT_ACC:
            raise OracleError("%s: not accumulator space" % what)
        if not addr & BIT_FULL:
            raise OracleError("%s: lacks full-C width" % what)
        base = addr & (BIT_FULL - 1)
        if base + DIM > acc_rows:
            raise OracleError("%s: accumulator rows exceed capacity" % what)
        return base

    for c in as_dicts(cmds):
        stats["instructions"] += 1
        kind = c["kind"]
        if kind == "config_ex":
            if c["dataflow"] != 1:
                raise OracleError("weight-stationary only")
            dataflow = 1
        elif kind == "config_ld":
            if c["slot"] not in (0, 1, 2) or c["scale"] != 1.0 or c["stride_bytes"] < 0:
                raise OracleError("unsupported config_ld")
            ld_stride[c["slot"]] = c["stride_bytes"]
        elif kind == "config_st":
            st_stride = c["stride_bytes"]
        elif kind == "mvin":
            stride = ld_stride.get(c["slot"])
            if stride is None:
                raise OracleError("mvin before config_ld")
            if c["cols"] != DIM or c["rows"] != DIM or c["buf"] not in ("A", "B"):
                raise OracleError("full tiles of A or B only")
            off = c["offset"]
            if not (0 <= off and off + (DIM - 1) * stride + DIM <= size[c["buf"]]):
                raise OracleError("mvin: dram range out of bounds")
            if not (0 <= c["spad_addr"] and c["spad_addr"] + DIM <= sp_rows):
                raise OracleError("mvin: scratchpad destination out of range")
            for r in range(DIM):
                spad[c["spad_addr"] + r] = src[c["buf"]][off + r * stride: off + r * stride + DIM].copy()
            in_flight += 1
        elif kind == "preload":
            pending_b = c["bd_spad_addr"]
            out_addr = c["out_addr"]
        elif kind == "compute":
            if dataflow != 1 or pending_b is None or out_addr is None:
                raise OracleError("compute without configuration and preload")
            if c["bd_spad_addr"] != GARBAGE:
                raise OracleError("compute requires garbage BD operand")
            if c["accumulated"]:
                if pending_b != GARBAGE or latched is None:
                    raise OracleError("compute_accumulated requires retained weights")
            else:
                if pending_b == GARBAGE:
                    raise OracleError("compute_preloaded requires an explicit B source")
                latched = spad_tile(pending_b, "compute preload B")
            a_tile = spad_tile(c["a_spad_addr"], "compute A")
            base = acc_base(out_addr, "compute output")
            prod = a_tile @ latched
            overwrite = not out_addr & BIT_ACCUMULATE
            for r in range(DIM):
                if overwrite:
                    row = prod[r].copy()
                    stats["overwrites"] += 1
                else:
                    if acc[base + r] is None:
                        raise OracleError("accumulation into uninitialized output")
                    row = acc[base + r] + prod[r]
                    stats["accumulates"] += 1
                if row.max() > INT32_MAX or row.min() < INT32_MIN:
                    raise OracleError("int32 accumulator overflow")
                acc[base + r] = row
            stats["macs"] += DIM * DIM * DIM
        elif kind == "mvout":
            if st_stride is None:
                raise OracleError("mvout before config_st")
            if c["cols"] != DIM or c["rows"] != DIM:
                raise OracleError("full tiles only")
            se = st_stride // 4
            if st_stride % 4 or se < n:
                raise OracleError("mvout stride invalid")
            off = c["buf_offset"]
            if not (0 <= off and off + (DIM - 1) * se + DIM <= m * n):
                raise OracleError("mvout: dram range out of bounds")
            base = acc_base(c["acc_addr"], "mvout source")
            for r in range(DIM):
                row = acc[base + r]
                if row is None:
                    raise OracleError("read of uninitialized accumulator")
                for col in range(DIM):
                    C[off + r * se + col] = int(row[col])
                    written[off + r * se + col] = True
            if in_flight > 0:
                in_flight -= 1
        elif kind == "fence":
            in_flight = 0
        else:
            raise OracleError("unknown command kind %r" % (kind,))
    if in_flight:
        raise OracleError("missing fence")
    if not all(written):
        raise OracleError("not every output element was written")
    return C, stats
