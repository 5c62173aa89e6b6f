"""Run and time a matmul loop nest — the runner side of the cpu_gemm path, on a B200.

Drop-in for the reference's specializations/cpu_gemm/runner.py.  `benchmark_matmul` (reference
:111-232) keeps its signature, its operand pattern (:150-151), its warm-up + `num_runs` timed
repetitions (:169-184), its four compared cells (:185-186, :216-223) and its result keys (:225-232);
what changes is that the nest is proved to be a GEMM (recognise.py) and executed by the hand-written
sm_100a fp32 kernel through the C ABI (vt_sgemm) instead of being emitted as C and compiled with
gcc.  `compile_and_run` (reference :65-108) still compiles and runs C text on the host, for callers
that use the emitter's output directly.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import tempfile
import time

import numpy as np

from .emit_c import emit_function, emit_test_harness  # noqa: F401  (part of the module's surface)
from .lower import parse_stmt
from .recognise import NotAMatmul, recognise_matmul

_OMP_BASE: tuple[str, list[str]] | None = None  # cached (compiler, OpenMP flags); None = not probed / none found
_OMP_PROBED = False


def _find_omp_base() -> tuple[str, list[str]] | None:
    """First compiler that compiles and links an OpenMP program: VERITAC_CC, gcc-16..gcc-12, gcc, clang."""
    names = [os.environ.get("VERITAC_CC")] + [f"gcc-{v}" for v in (16, 15, 14, 13, 12)] + ["gcc", "clang"]
    flags = ["-fopenmp", "-O2"]
    if shutil.which("xcrun"):
        try:
            sdk = subprocess.run(["xcrun", "--show-sdk-path"], capture_output=True, text=True).stdout.strip()
        except Exception:
            sdk = ""
        if sdk:
            flags += ["-isysroot", sdk, "-I", f"{sdk}/usr/include"]
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "probe.c")
        with open(src, "w") as fh:
            fh.write("int main(void){return 0;}\n")
        for cc in names:
            if not cc:
                continue
            try:
                r = subprocess.run([cc] + flags + ["-o", os.path.join(tmp, "probe"), src], capture_output=True,
                                   text=True, timeout=20)
            except (FileNotFoundError, subprocess.TimeoutExpired):
                continue
            if r.returncode == 0:
                return cc, flags
    return None


def compile_and_run(c_code: str, timeout: float = 30.0) -> tuple[str, float]:
    """Compile C text with the host compiler, run it, return (stdout, elapsed seconds).

    RuntimeError on a compile or run failure, like the reference.  Without an OpenMP compiler the
    pragmas are inert and the program still computes the same values.
    """
    global _OMP_BASE, _OMP_PROBED
    if not _OMP_PROBED:
        _OMP_BASE = _find_omp_base()
        _OMP_PROBED = True
    with tempfile.TemporaryDirectory() as tmp:
        src, exe = os.path.join(tmp, "kernel.c"), os.path.join(tmp, "kernel")
        with open(src, "w") as fh:
            fh.write(c_code)
        if _OMP_BASE is not None:
            cmd = [_OMP_BASE[0]] + _OMP_BASE[1] + ["-o", exe, src, "-lm"]
        else:
            cmd = [os.environ.get("VERITAC_CC", "clang"), "-O2", "-o", exe, src, "-lm"]
        built = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
        if built.returncode != 0:
            raise RuntimeError(f"Compilation failed:\n{built.stderr}")
        t0 = time.perf_counter()
        ran = subprocess.run([exe], capture_output=True, text=True, timeout=timeout)
        elapsed = time.perf_counter() - t0
        if ran.returncode != 0:
            raise RuntimeError(f"Execution failed:\n{ran.stderr}")
        return ran.stdout, elapsed


def matmul_operands(M: int, K: int, N: int, dtype=np.float32):
    """The runner's operands as dense row-major matrices: A[i,k] = (i*K+k) % 7, B[k,j] = (k*N+j) % 5."""
    a = (np.arange(M * K, dtype=np.int64) % 7).astype(dtype).reshape(M, K)
    b = (np.arange(K * N, dtype=np.int64) % 5).astype(dtype).reshape(K, N)
    return a, b


def schedule_hint(shape: dict) -> dict:
    """What a recognised nest's schedule says about tiling, in this back end's terms.

    The tile tactic leaves `<v>_outer` / `<v>_inner` loops (VeriTac/Tactic/Tile.lean:284-321); the innermost loop
    of the row role and of the column role give the tile a CPU schedule meant to keep in cache, which on the GPU
    is the CTA tile: up to 32 -> the 32x32 kernel, up to 64 -> the 64x64 kernel, beyond -> the 128x128 kernel.
    A nest without a split row or column loop gives no hint (None).  The annotations are carried along for the
    caller to show; on the GPU every output cell is computed in parallel whatever they say.
    """
    from ... import _native as nv

    inner = {}
    for var, extent, ann, role in shape["loops"]:
        inner[role] = (var, extent)                      # the last loop of each role is its innermost
    split = {role: sum(1 for l in shape["loops"] if l[3] == role) > 1 for role in ("i", "j", "k")}
    tile_m = inner["i"][1] if split["i"] else None
    tile_n = inner["j"][1] if split["j"] else None
    variant = None
    if tile_m or tile_n:
        side = max(tile_m or 0, tile_n or 0)
        variant = nv.VT_SGEMM_TILE32 if side <= 32 else nv.VT_SGEMM_TILE64 if side <= 64 else nv.VT_SGEMM_TILE128
    return {"tile_m": tile_m, "tile_n": tile_n, "variant": variant,
            "parallel": [v for v, _n, ann, _r in shape["loops"] if ann == "parallel"],
            "vectorize": [v for v, _n, ann, _r in shape["loops"] if ann == "vectorize"]}


def benchmark_matmul(stmt_json: dict, M: int, K: int, N: int, num_runs: int = 5, time_hint: bool = False) -> dict:
    """Time a matmul loop nest on the GPU against numpy and check its result.

    Args are the reference's: the loop-nest JSON, then M, K, N (note the order), then the number of
    timed repetitions.  Raises ValueError for malformed JSON (as parse_stmt does) and RuntimeError
    when the nest is not a GEMM this back end can run or the device call fails.

    Returns the reference's keys — c_time_ms (average device time of one matmul, operands resident
    in HBM, the counterpart of the reference timing `matmul()` on resident host buffers),
    numpy_time_ms, speedup, correct (the same four cells within 1e-6), c_first_values,
    np_first_values — plus e2e_time_ms (one call with host buffers, copies included),
    rel_frobenius_error of the whole result against float64, `kernel` (the kernel the library chose for the
    shape) and `schedule_hint` (schedule_hint() of the nest).  The timed call always uses the library's own
    choice; with `time_hint` the kernel the schedule's tile sizes point at is timed as well (`hint_time_ms`,
    `hint_kernel`), so that a caller can see what honouring the schedule would have cost.
    """
    stmt = parse_stmt(stmt_json)
    try:
        shape = recognise_matmul(stmt, M, K, N)
    except NotAMatmul as exc:
        raise RuntimeError(f"loop nest is not a GEMM the B200 back end can execute: {exc}") from exc
    hint = schedule_hint(shape)

    import torch  # device memory, stream and events only

    from ... import _native as nv

    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: the B200 back end has no CPU fallback")
    a32, b32 = matmul_operands(M, K, N, np.float32)
    dev = torch.cuda.current_device()
    stream = nv.torch_stream()
    try:
        dA = torch.from_numpy(a32).to("cuda")
        dB = torch.from_numpy(b32).to("cuda")
        dC = torch.zeros((M, N), dtype=torch.float32, device="cuda")
        nv.sgemm(dA, dB, dC, M, N, K, dev=dev, where=nv.VT_DEVICE, stream=stream)  # warm-up
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        total_ms = 0.0
        for _ in range(num_runs):
            dC.zero_()
            start.record()
            nv.sgemm(dA, dB, dC, M, N, K, dev=dev, where=nv.VT_DEVICE, stream=stream)
            stop.record()
            stop.synchronize()
            total_ms += start.elapsed_time(stop)
        nv.sync(dev, stream)
        c_host = dC.cpu().numpy()
        chosen = nv.sgemm_auto_variant(M, N, K, dev=dev)
        hint_ms = None
        if time_hint and hint["variant"] is not None and num_runs:
            tileable = hint["variant"] != nv.VT_SGEMM_TILE32 or (N % 4 == 0 and K % 4 == 0)
            if tileable:
                dH = torch.zeros((M, N), dtype=torch.float32, device="cuda")
                nv.sgemm(dA, dB, dH, M, N, K, dev=dev, variant=hint["variant"], where=nv.VT_DEVICE, stream=stream)
                hint_total = 0.0
                for _ in range(num_runs):            # timed exactly as the library's choice above
                    dH.zero_()
                    start.record()
                    nv.sgemm(dA, dB, dH, M, N, K, dev=dev, variant=hint["variant"], where=nv.VT_DEVICE, stream=stream)
                    stop.record()
                    stop.synchronize()
                    hint_total += start.elapsed_time(stop)
                hint_ms = hint_total / num_runs
                nv.sync(dev, stream)
        # once more through host buffers: what a caller without device memory pays
        c_e2e = np.empty((M, N), dtype=np.float32)
        t0 = time.perf_counter()
        nv.sgemm(a32, b32, c_e2e, M, N, K, dev=dev, where=nv.VT_HOST)
        e2e_ms = (time.perf_counter() - t0) * 1000.0
    except nv.NativeError as exc:
        raise RuntimeError(f"Execution failed:\n{exc}") from exc
    c_time_ms = total_ms / num_runs if num_runs else None

    a64, b64 = a32.astype(np.float64), b32.astype(np.float64)
    t0 = time.perf_counter()
    for _ in range(num_runs):
        c_np = a64 @ b64
    np_time_ms = ((time.perf_counter() - t0) / num_runs) * 1000.0 if num_runs else 0.0
    if not num_runs:
        c_np = a64 @ b64

    cells = [(0, 0), (1, 0), (M - 1, 0), (M - 1, N - 1)]  # flat 0, 1000, 1000(M-1), 1000(M-1)+(N-1)
    c_values = [float(c_host[r, c]) if r < M and c < N else float("nan") for r, c in cells]
    expected = [float(c_np[r, c]) if r < M and c < N else float("nan") for r, c in cells]
    correct = all(abs(c_values[i] - expected[i]) < 1e-6 for i in range(4)) and bool(np.array_equal(c_host, c_e2e))
    denom = float(np.linalg.norm(c_np))
    rel = float(np.linalg.norm(c_host.astype(np.float64) - c_np) / denom) if denom else 0.0
    return {
        "c_time_ms": c_time_ms,
        "numpy_time_ms": np_time_ms,
        "speedup": np_time_ms / c_time_ms if c_time_ms else 0,
        "correct": correct,
        "c_first_values": c_values,
        "np_first_values": expected,
        "e2e_time_ms": e2e_ms,
        "rel_frobenius_error": rel,
        "kernel": nv.SGEMM_VARIANT_NAMES.get(chosen, str(chosen)),
        "schedule_hint": hint,
        "hint_kernel": nv.SGEMM_VARIANT_NAMES.get(hint["variant"]) if hint["variant"] is not None else None,
        "hint_time_ms": hint_ms,
    }
