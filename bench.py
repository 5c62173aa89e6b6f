#!/usr/bin/env python3
"""Benchmark of the B200 GEMM back end on the reference's headline workload.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One JSON line on stdout (rank 0).  A *step* is one pass of the hot path over one batch of synthetic
input: one GEMM of the named shape.  Default workload: exact int8 x int8 -> int32 GEMM with
M = N = K = 8192; with N GPUs the 8192 rows of A and C are split over the ranks (rank r owns rows
[r*M/N, (r+1)*M/N), strong scaling) and B is broadcast from rank 0 over NCCL before timing.  There is
no data-path collective.  `--scaling weak` gives every rank the whole shape instead.

  value      whole-job throughput, operands resident in HBM, CUDA-event time on the launching
             stream, max over ranks
  e2e        same metric through the C ABI with pinned HOST buffers: host->device copies of A and B
             and the device->host copy of C are inside the timed region of every step (with N > 1, B
             crosses the host link on rank 0 only and reaches the other GPUs by the broadcast, also
             inside the timed region); link_floor_ms = plain copies of the same bytes, no compute
  parity     after the timed regions every rank checks sampled rows of its C, from the device-resident
             run and from the host-buffer run, against the exact product; ok = all ranks passed
  roofline   achieved = algorithmic ops (or bytes) per launch / average launch duration of the
             timed region; peak from MEASURED_PEAKS.json (fallback stated if absent)
  also       the other named workloads, each timed like the headline (fp32 256^3 and 640^3, fp32 8192^3 by
             the automatic choice and by the FFMA kernel, fp32 16 x 8192 x 8192, the batched B-reuse int8
             workload), short launches first, a quarter of a second apart; workloads of less than 30 us
             per step also as one CUDA graph of the 20 calls (`graph_replay`)
  cpu_baseline  the oracle's OpenMP C restatement of the reference's CPU arithmetic, timed on this
             host's cores on a bounded sample of the same workload (N = 1 only)

`--impl reference` times that CPU restatement alone, with every host thread, on bounded samples of
the same workload, and prints the same line shape with "impl": "reference".
"""
from __future__ import annotations

import argparse
import math
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

NOMINAL_INT8_TOPS = 4500.0     # dense int8, NVIDIA's B200 figure
NOMINAL_FP32_TFLOPS = 74.45    # 148 SMs x 128 FMA lanes x 2 x 1.965 GHz
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel, constants typed in
# from ncu captures of these workloads on one GPU (a run of this script cannot measure them); None where no
# capture was taken.
NCU_TRAFFIC_BYTES = {"sgemm_skinny": 273.9e6, "sgemm_panel_128": 282.9e6, "sgemm_tall_16": 275.8e6, "i8_8192": 496.1e6, "i8_batched_32": 654.4e6, "i8_batched": 8 * 654.4e6}

WORKLOADS = {
    # name: (kind, M, N, K, batch)
    "i8_8192": ("i8", 8192, 8192, 8192, 1),
    "i8_64": ("i8", 64, 64, 64, 1),
    "i8_shard_2048": ("i8", 2048, 8192, 8192, 1),         # one GPU's rows of the 8192^3 product on 4 GPUs
    "i8_shard_1024": ("i8", 1024, 8192, 8192, 1),         # ... on 8 GPUs
    "i8_batched": ("i8b", 1024, 4096, 4096, 256),
    "i8_batched_32": ("i8b", 1024, 4096, 4096, 32),      # one GPU's share of the batched workload on 8 GPUs
    "sgemm_8192": ("f32", 8192, 8192, 8192, 1),
    "sgemm_256": ("f32", 256, 256, 256, 1),
    "sgemm_640": ("f32", 640, 640, 640, 1),               # a mid-sized product: FFMA with K split over a cluster
    "sgemm_skinny": ("f32", 16, 8192, 8192, 1),
    "sgemm_panel_64": ("f32", 64, 8192, 8192, 1),         # few rows against a large B: the row-panel kernel
    "sgemm_panel_128": ("f32", 128, 8192, 8192, 1),
    "sgemm_tall_16": ("f32", 8192, 16, 8192, 1),          # few columns against a large A: the tall form
}


def load_peaks():
    path = REPO / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            return json.loads(path.read_text()), "measured"
        except ValueError:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """SM clock, power and clock-event reasons of one GPU, read through NVML by a polling thread; only samples taken between mark_begin() and mark_end() (the timed region)
    count.  Falls back to an `nvidia-smi -lms` child when NVML cannot be loaded."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    REASON_BITS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
                   ("sw_power_cap", 0x4))

    def __init__(self, index: int, uuid: str | None = None):
        self.index = index
        self.uuid = uuid
        self.samples: list[tuple] = []       # (host time, sm MHz, reason mask, watts)
        self.rows: list[list[str]] = []      # nvidia-smi fallback
        self.proc = None
        self.thread = None
        self.nvml = None
        self.handle = None
        self.max_mhz = None
        self.running = False
        self.t_begin = self.t_end = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + self.uuid).encode()) if self.uuid else None
            except Exception:
                self.handle = None
            if self.handle is None:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.running = True
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _poll(self):
        nv, h = self.nvml, self.handle
        while self.running:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                watts = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
            except Exception:
                break
            self.samples.append((time.perf_counter(), float(mhz), int(mask), watts))
            time.sleep(0.0005)   # leave the interpreter to the launching thread

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([time.perf_counter()] + [x.strip() for x in line.split(",")])

    def mark_begin(self):
        self.t_begin = time.perf_counter()

    def mark_end(self):
        self.t_end = time.perf_counter()

    def _inside(self, t):
        return self.t_begin is None or self.t_end is None or self.t_begin <= t <= self.t_end

    def window(self, t0: float, t1: float) -> dict | None:
        """Median clock, reasons and peak power of the NVML samples taken in [t0, t1] (None without NVML)."""
        if self.nvml is None:
            return None
        inside = [x for x in list(self.samples) if t0 <= x[0] <= t1]
        sm = [x[1] for x in inside]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_mhz_min": min(sm) if sm else None,
                "reasons": sorted({name for x in inside for name, bit in self.REASON_BITS if x[2] & bit}),
                "samples": len(sm), "power_w_max": max(x[3] for x in inside) if inside else None}

    def stop(self) -> dict:
        if self.nvml is not None:
            self.running = False
            self.thread.join(timeout=2)
            inside = [x for x in self.samples if self._inside(x[0])]
            reasons = sorted({name for x in inside for name, bit in self.REASON_BITS if x[2] & bit})
            sm = [x[1] for x in inside]
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz, "reasons": reasons,
                    "samples": len(sm), "sm_mhz_min": min(sm) if sm else None,
                    "power_w_max": max(x[3] for x in inside) if inside else None,
                    "source": "NVML polled during the timed region"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["NVML and nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        rows = [r for r in self.rows if self._inside(r[0])] or self.rows
        for r in rows:
            r = r[1:]
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, flag in zip(names, r[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi -lms 20"}


# ---------------------------------------------------------------------------------------------
# CPU baseline: the oracle's C restatement on a bounded sample (checker code, timed, never shipped)
# ---------------------------------------------------------------------------------------------
def _oracle_lib():
    sys.path.insert(0, str(REPO / "oracle"))
    import build_oracle

    lib = ctypes.CDLL(str(build_oracle.build()))
    i64, vp = ctypes.c_long, ctypes.c_void_p
    lib.oracle_i8_tiled_ref.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64]
    for name in ("oracle_sgemm_tuned", "oracle_dgemm_tuned", "oracle_sgemm_naive"):
        getattr(lib, name).argtypes = [vp, vp, vp, i64, i64, i64]
    lib.oracle_threads.restype = ctypes.c_int
    return lib


class CpuArm:
    """Times rows [0, R) of the workload's product on the host cores; R is sized from a probe so one
    sample takes about `seconds`.  Rows are independent, so ops/s of the sample is ops/s of the job."""

    kind_label = "port"

    def __init__(self, kind, M, N, K, seed):
        import numpy as np

        self.np = np
        self.kind, self.M, self.N, self.K = kind, M, N, K
        self.lib = _oracle_lib()
        try:
            allowed = len(os.sched_getaffinity(0))
        except AttributeError:
            allowed = os.cpu_count() or 1
        self.lib.oracle_set_threads(ctypes.c_int(allowed))   # not whatever OMP_NUM_THREADS the launcher exported
        self.threads = int(self.lib.oracle_threads())
        # The README schedule tiles i1 by 32, which the tile tactic refuses when 32 does not divide N; the untuned
        # nest of make_matmul_stmt (one thread) is then what the reference has for the shape.
        self.untuned = kind == "f32" and N % 32 != 0
        if self.untuned:
            self.threads = 1
        rng = np.random.default_rng(seed)
        self.block = 16 if kind != "f32" else 32
        self.unit = self.block * self.threads            # rows that keep every thread busy
        self.max_rows = max(self.unit, min(M, 64 * self.unit)) // self.block * self.block
        self.max_rows = min(self.max_rows, M - M % self.block) or self.block
        if kind == "f32":
            self.A = (rng.random((self.max_rows, K), dtype=np.float32) * 2 - 1)
            self.B = (rng.random((K, N), dtype=np.float32) * 2 - 1)
            self.C = np.zeros((self.max_rows, N), dtype=np.float32)
        else:
            self.A = rng.integers(-128, 128, (self.max_rows, K), dtype=np.int8)
            self.B = rng.integers(-128, 128, (K, N), dtype=np.int8)
            self.C = np.zeros((self.max_rows, N), dtype=np.int32)

    def run_rows(self, rows: int) -> float:
        t0 = time.perf_counter()
        if self.kind == "f32":
            self.C[:rows] = 0
            fn = self.lib.oracle_sgemm_naive if self.untuned else self.lib.oracle_sgemm_tuned
            fn(self.A.ctypes.data, self.B.ctypes.data, self.C.ctypes.data, rows, self.N, self.K)
        else:
            self.lib.oracle_i8_tiled_ref(self.A.ctypes.data, self.B.ctypes.data, self.C.ctypes.data, rows, self.N,
                                         self.K, 0, rows)
        return time.perf_counter() - t0

    def size_sample(self, seconds: float) -> int:
        probe = min(self.unit, self.max_rows)
        t = self.run_rows(probe)
        rows = int(probe * seconds / max(t, 1e-6)) // self.block * self.block
        return max(self.block, min(rows, self.max_rows))

    def ops(self, rows: int) -> float:
        return 2.0 * rows * self.N * self.K

    def describe(self, rows: int) -> str:
        what = ("C restatement of the untuned generated fp32 nest (tile 32 does not divide N), one thread"
                if self.untuned else
                "OpenMP C restatement of the generated tile(32)x2/reorder/simd/parallel fp32 nest"
                if self.kind == "f32" else
                "OpenMP C restatement of the reference's int8 tile loop (baseline i,j,k order)")
        return "%s; rows [0,%d) of the %dx%dx%d product (all of B)" % (what, rows, self.M, self.N, self.K)


class GeneratedCArm:
    """The reference's own generated OpenMP C for a whole M = N = K product: `matmul()` printed by its
    unmodified emitter for the README schedule and compiled ahead of time into oracle/_ref/ (doubles, row
    stride 1000, as the reference lays its buffers out).  One unit of work is the whole product, timed the
    way the reference's runner times it (clear C, call matmul)."""

    kind_label = "reference"

    def __init__(self, path, dim):
        import numpy as np

        self.np, self.dim = np, dim
        self.lib = ctypes.CDLL(str(path))
        self.lib.matmul.argtypes = [ctypes.c_void_p] * 3
        try:
            allowed = len(os.sched_getaffinity(0))
        except AttributeError:
            allowed = os.cpu_count() or 1
        try:                                           # same OpenMP runtime as the loaded object
            gomp = ctypes.CDLL("libgomp.so.1")
            gomp.omp_set_num_threads(ctypes.c_int(allowed))
            gomp.omp_get_max_threads.restype = ctypes.c_int
            self.threads = int(gomp.omp_get_max_threads())
        except OSError:
            self.threads = int(os.environ.get("OMP_NUM_THREADS", allowed))
        rng = np.random.default_rng(20260917)
        self.A = np.zeros((dim, 1000)); self.B = np.zeros((dim, 1000)); self.C = np.zeros((dim, 1000))
        self.A[:, :dim] = rng.random((dim, dim)) * 2 - 1
        self.B[:, :dim] = rng.random((dim, dim)) * 2 - 1

    def run_rows(self, reps: int) -> float:
        t0 = time.perf_counter()
        for _ in range(reps):
            self.C[:] = 0
            self.lib.matmul(self.A.ctypes.data, self.B.ctypes.data, self.C.ctypes.data)
        return time.perf_counter() - t0

    def size_sample(self, seconds: float) -> int:
        self.run_rows(2)
        t = self.run_rows(5) / 5
        return max(5, int(min(seconds, 10.0) / max(t, 1e-6)))

    def ops(self, reps: int) -> float:
        return 2.0 * self.dim ** 3 * reps

    def describe(self, reps: int) -> str:
        return ("matmul() as printed by the reference's emitter for the README schedule (double, row stride 1000, "
                "OpenMP), %d whole %d^3 products" % (reps, self.dim))


def make_cpu_arm(args, kind, M, N, K):
    """The reference's generated C where it was built for this exact shape, else the C restatement."""
    ref = REPO / "oracle" / "_ref" / ("matmul_%d_readme.so" % M)
    if kind == "f32" and M == N == K and ref.is_file():
        return GeneratedCArm(ref, M)
    return CpuArm(kind, M, N, K, seed=20260917)


def run_reference_arm(args, kind, M, N, K, metric, unit):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    arm = make_cpu_arm(args, kind, M, N, K)
    steps, warm = max(1, args.steps), max(0, args.warmup)
    rows = arm.size_sample(min(8.0, 120.0 / (steps + warm)))
    for _ in range(warm):
        arm.run_rows(rows)
    total = 0.0
    for _ in range(steps):
        total += arm.run_rows(rows)
    value = arm.ops(rows) * steps / total / 1e12
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": total / steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32" if kind == "f32" else "s8->s32", "data": "synthetic",
        "config": {"workload": args.workload, "M_per_gpu": M, "N": N, "K": K, "global_M": M,
                   "note": "CPU arm: each step is a bounded row sample of the workload on the host cores"},
        "cpu_baseline": {"value": value, "unit": unit, "cores": arm.threads, "kind": arm.kind_label,
                         "sample": arm.describe(rows)},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
PANEL_WORKLOADS = ("sgemm_skinny", "sgemm_panel_64", "sgemm_panel_128", "sgemm_tall_16")


def roofline_for(workload, kind, rows, N, K, launch_ms, peaks, peaks_src, sgemm_variant, nv):
    """Roofline object of the dominant kernel of one rank's launch (see the module docstring)."""
    ops_per_launch = 2.0 * rows * N * K
    algo_bytes = (K * N + rows * K + rows * N) * 4.0
    tf32x3_peak = peaks["bf16_tflops"] / 2.0 / 3.0       # three TF32 MMAs per fp32 product; TF32 at half the bf16 rate
    panel = workload in PANEL_WORKLOADS
    if panel and algo_bytes / (peaks["hbm_gbs"] * 1e9) >= ops_per_launch / (tf32x3_peak * 1e12):
        achieved = algo_bytes / (launch_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "peak_source": "%s hbm_gbs" % peaks_src}
    elif panel:
        # enough rows that the three TF32 MMAs per product take longer than streaming B
        achieved = ops_per_launch / (launch_ms * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": tf32x3_peak, "unit": "TFLOP/s",
                "frac": achieved / tf32x3_peak,
                "peak_source": "%s bf16_tflops / 2 (TF32 rate) / 3 (MMAs per fp32 product); streaming B at %s hbm_gbs "
                               "would take less" % (peaks_src, peaks_src),
                "hbm_gbs_achieved": algo_bytes / (launch_ms * 1e-3) / 1e9}
    elif kind == "f32":
        achieved = ops_per_launch / (launch_ms * 1e-3) / 1e12
        tensor_path = sgemm_variant == nv.VT_SGEMM_TF32X3 or (
            sgemm_variant == nv.VT_SGEMM_AUTO and rows >= 256 and N >= 256 and K >= 256
            and float(rows) * N * K >= 5.0e8 and N % 4 == 0 and K % 4 == 0)
        if tensor_path:
            roof = {"bound": "tensor", "achieved": achieved, "peak": tf32x3_peak, "unit": "TFLOP/s",
                    "frac": achieved / tf32x3_peak,
                    "peak_source": "%s bf16_tflops / 2 (TF32 rate) / 3 (MMAs per fp32 product); the step also holds the "
                                   "pass that writes the lo parts" % peaks_src,
                    "vs_ffma_pipe_74.45": achieved / NOMINAL_FP32_TFLOPS}
        else:
            roof = {"bound": "fp32", "achieved": achieved, "peak": NOMINAL_FP32_TFLOPS, "unit": "TFLOP/s",
                    "frac": achieved / NOMINAL_FP32_TFLOPS,
                    "peak_source": "FFMA pipe at clocks.max.sm: 148 SMs x 128 lanes x 2 x 1.965 GHz (no fp32 SIMT "
                                   "figure in MEASURED_PEAKS.json)"}
    else:
        achieved = ops_per_launch / (launch_ms * 1e-3) / 1e12
        peak = 2.0 * peaks["bf16_tflops"]
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s", "frac": achieved / peak,
                "peak_source": "2 x %s bf16_tflops (kind::i8 issues at twice the bf16 rate)" % peaks_src,
                "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS}
    roof["traffic"] = NCU_TRAFFIC_BYTES.get(workload)
    roof["traffic_source"] = ("constant from an ncu capture of this workload on one GPU, not measured by this run"
                              if roof["traffic"] is not None else None)
    roof["launch_ms"] = launch_ms
    return roof


class Job:
    """One workload on this rank: operands in HBM, the device-resident step, timing, the parity check."""

    def __init__(self, ctx, workload, scaling, i8_variant=0, sgemm_variant=0):
        torch, nv, sharding = ctx["torch"], ctx["nv"], ctx["sharding"]
        self.ctx, self.workload = ctx, workload
        self.kind, self.M, self.N, self.K, self.batch = WORKLOADS[workload]
        self.i8_variant, self.sgemm_variant = i8_variant, sgemm_variant
        rank, world = ctx["rank"], ctx["world"]
        total = self.M * self.batch
        # too few rows to split (or a shape that is about one GPU's grid of tiles): every rank runs the whole shape
        self.replicas = world > 1 and (total < 64 * world or workload == "sgemm_640")
        if scaling == "weak" or world == 1 or self.replicas:
            self.rows = total
        else:
            r0, r1 = sharding.row_shard(total, world, rank, align=self.M if self.kind == "i8b" else 16)
            self.rows = r1 - r0
        gen = torch.Generator(device="cuda").manual_seed(20260917 + rank + 1000 * (sorted(WORKLOADS).index(workload) + 1))
        self.gen = gen
        N, K, rows = self.N, self.K, self.rows
        if self.kind == "f32":
            self.A = torch.rand((rows, K), device="cuda", generator=gen) * 2 - 1
            self.B = torch.rand((K, N), device="cuda", generator=gen) * 2 - 1
            self.C = torch.zeros((rows, N), device="cuda")
            self.elem_in, self.elem_out = 4, 4
        else:
            self.A = torch.randint(-128, 128, (rows, K), dtype=torch.int8, device="cuda", generator=gen)
            self.B = torch.randint(-128, 128, (K, N), dtype=torch.int8, device="cuda", generator=gen)
            self.C = torch.empty((rows, N), dtype=torch.int32, device="cuda")
            self.elem_in, self.elem_out = 1, 4
        # Operands: A differs per rank (its own row block); B is rank 0's, delivered by broadcast.
        sharding.replicate_from_rank0(self.B)
        self.total_rows = ctx["sum"](float(rows)) if not self.replicas else float(rows)

    def step(self):
        nv, dev, st = self.ctx["nv"], self.ctx["dev"], self.ctx["st"]
        if self.rows == 0:
            return
        if self.kind == "f32":
            nv.sgemm(self.A, self.B, self.C, self.rows, self.N, self.K, dev=dev, variant=self.sgemm_variant,
                     where=nv.VT_DEVICE, stream=st)
        elif self.kind == "i8b":
            nv.i8gemm_shared_b(self.A, self.B, self.C, self.rows // self.M, self.M, self.N, self.K, dev=dev, acc_rows=16,
                               where=nv.VT_DEVICE, stream=st)
        else:
            nv.i8gemm(self.A, self.B, self.C, self.rows, self.N, self.K, dev=dev, variant=self.i8_variant,
                      where=nv.VT_DEVICE, stream=st)

    def timed(self, steps, warm, sampler=None):
        """(ms per step: CUDA events on the launching stream, max over ranks; kernel launches of this rank)."""
        torch, nv, ctx = self.ctx["torch"], self.ctx["nv"], self.ctx
        for _ in range(warm):
            self.step()
        nv.sync(ctx["dev"], ctx["st"])
        ctx["barrier"]()
        launches0 = nv.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx["barrier"]()
        if sampler:
            sampler.mark_begin()
        e0.record()
        for _ in range(steps):
            self.step()
        e1.record()
        ctx["barrier"]()
        if sampler:
            sampler.mark_end()
        ms = ctx["max"](e0.elapsed_time(e1)) / steps
        launches = nv.launch_count() - launches0
        nv.sync(ctx["dev"], ctx["st"])
        return ms, launches

    def graph_ms(self, steps):
        """ms per step with the `steps` calls captured once into a CUDA graph and replayed: what a launch-bound
        workload costs when the host's per-call work (argument checks, tensor maps, the launch itself) is paid at
        capture time.  CUDA events around one replay, max over ranks."""
        torch, ctx = self.ctx["torch"], self.ctx
        side = torch.cuda.Stream()
        saved = ctx["st"]
        ctx["st"] = int(side.cuda_stream)
        try:
            with torch.cuda.stream(side):
                self.step()
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(steps):
                    self.step()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(side):
                graph.replay()
                e0.record()
                graph.replay()
                e1.record()
            side.synchronize()
            ctx["nv"].sync(ctx["dev"], ctx["st"])
            return ctx["max"](e0.elapsed_time(e1)) / steps
        finally:
            ctx["st"] = saved

    def value(self, ms_per_step):
        """Whole-job throughput in T(FL)OPS; replicas count once (every rank does the same whole product)."""
        return 2.0 * self.total_rows * self.N * self.K / (ms_per_step * 1e-3) / 1e12

    def check(self, C, samples=32):
        """Sampled rows of this rank's C against the exact product.  int8: float64 matmul of the sampled rows is exact
        (|sum| < 2^53) and every bit must agree; fp32: relative Frobenius error of the sampled rows against float64,
        bound 1e-5."""
        torch = self.ctx["torch"]
        if self.rows == 0:
            return {"ok": True, "rows_checked": 0}
        idx = torch.randint(0, self.rows, (min(samples, self.rows),), device="cuda", generator=self.gen)
        got = C[idx.cpu()] if C.device.type == "cpu" else C[idx]
        got = got.cuda()
        exact = self.A[idx].double() @ self.B.double()
        if self.kind == "f32":
            err = float(torch.linalg.norm(got.double() - exact) / torch.linalg.norm(exact))
            return {"ok": bool(err <= 1e-5), "rows_checked": int(idx.numel()), "rel_frobenius": err, "bound": 1e-5}
        bad = int((got.to(torch.int64) != exact.to(torch.int64)).sum().item())
        return {"ok": bad == 0, "rows_checked": int(idx.numel()), "cells_differing": bad}

    def release(self):
        self.A = self.B = self.C = None
        self.ctx["torch"].cuda.empty_cache()


def run_gpu_arm(args, kind, M, N, K, batch, metric, unit):
    import torch
    import torch.distributed as dist

    from veritac_b200 import _native as nv
    from veritac_b200 import build, sharding

    build.build()
    t_init0 = time.perf_counter()
    rank, world, local = sharding.init_process_group()
    if world != args.gpus:
        if rank == 0:
            sys.stderr.write("bench: --gpus %d but WORLD_SIZE is %d (launch with torchrun)\n" % (args.gpus, world))
        if args.gpus != 1:
            return 2
    if not torch.cuda.is_available():
        sys.stderr.write("bench: no CUDA device; the GPU arm has no CPU fallback\n")
        return 2
    torch.cuda.set_device(local)
    dev = local
    peaks, peaks_src = load_peaks()
    steps, warm = max(1, args.steps), max(3, args.warmup)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_scalar(x, op):
        if world == 1:
            return float(x)
        t = torch.tensor([float(x)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=op)
        return float(t.item())

    ctx = {"torch": torch, "nv": nv, "sharding": sharding, "rank": rank, "world": world, "dev": dev,
           "st": nv.torch_stream(), "barrier": barrier,
           "max": lambda x: reduce_scalar(x, dist.ReduceOp.MAX), "sum": lambda x: reduce_scalar(x, dist.ReduceOp.SUM),
           "min": lambda x: reduce_scalar(x, dist.ReduceOp.MIN)}

    # ---- communicator: created by the first collective; timed apart from the broadcast of B ----
    comm_init_ms = bcast_ms_warm = None
    if world > 1:
        tiny = torch.zeros(1, device="cuda")
        dist.broadcast(tiny, src=0)
        torch.cuda.synchronize()
        comm_init_ms = (time.perf_counter() - t_init0) * 1e3

    job = Job(ctx, args.workload, args.scaling, args.i8_variant, args.sgemm_variant)
    rows, global_rows = job.rows, int(job.total_rows)
    if world > 1:
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        b0.record()
        sharding.replicate_from_rank0(job.B)
        b1.record()
        torch.cuda.synchronize()
        bcast_ms_warm = ctx["max"](b0.elapsed_time(b1))

    try:
        gpu_uuid = str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        gpu_uuid = None
    sampler = ClockSampler(local, gpu_uuid)
    if rank == 0:
        sampler.start()
        time.sleep(0.05)
    ms_per_step, launches = job.timed(steps, warm, sampler)
    value = job.value(ms_per_step)

    # ---- parity of the device-resident run: this rank's C as the timed steps left it ----
    parity_device = job.check(job.C)

    # ---- end to end through the C ABI with pinned host buffers ----
    # One GPU: A, B and C are host buffers of one vt_* call.  Several GPUs, int8: B exists in rank 0's host memory
    # only; rank 0 copies it in, the broadcast carries it to the other GPUs, and every rank's call takes its rows
    # of A from and returns its rows of C to host memory (VT_HOST_AC_DEVICE_B).  All of that is inside the timed
    # region of every step.
    e2e = {"value": None, "unit": unit, "h2d_bytes_per_step": None, "d2h_bytes_per_step": None}
    parity_host = None
    if not args.no_e2e:
        e2e_steps = max(2, min(steps, 5))
        hA = torch.empty((rows, K), dtype=job.A.dtype).pin_memory()
        hC = torch.empty((rows, N), dtype=job.C.dtype).pin_memory()
        hA.copy_(job.A)
        shared_b = world > 1 and kind != "f32" and not job.replicas
        hB = torch.empty((K, N), dtype=job.B.dtype).pin_memory() if (rank == 0 or not shared_b) else None
        if hB is not None:
            hB.copy_(job.B)
        # B in column blocks, so that the first columns of C leave while later blocks of B still arrive
        streamed = shared_b and kind == "i8"
        blocks = sharding.column_blocks(N, 4) if streamed else None
        dA_stream = torch.empty_like(job.A) if streamed else None
        dB = ([torch.empty((K, cols), dtype=job.B.dtype, device="cuda") for _c0, cols in blocks] if streamed
              else torch.empty_like(job.B) if shared_b else None)
        ready = [torch.cuda.Event() for _ in blocks] if streamed else None

        def host_call(a, b, c, where):
            if rows == 0:
                return
            if kind == "f32":
                nv.sgemm(a, b, c, rows, N, K, dev=dev, where=where)
            elif kind == "i8b":
                nv.i8gemm_shared_b(a, b, c, rows // M, M, N, K, dev=dev, acc_rows=16, where=where, stream=ctx["st"])
            else:
                nv.i8gemm(a, b, c, rows, N, K, dev=dev, where=where, stream=ctx["st"])

        def stage_block(j, buf, c0, cols):
            nv.i8_stage_b_block(buf, hB, K, N, c0, cols, dev=dev, stream=ctx["st"])

        def mark_ready(j):
            ready[j].record()
            return ready[j]

        def e2e_step():
            if streamed:
                # this rank's rows of A go first, so that they do not queue behind B on the host link
                dA_stream.copy_(hA, non_blocking=True)
                sharding.run_row_sharded_streamed(
                    stage_block, lambda a, bs, evs, c: nv.i8gemm_rows_streamed_b(a, bs, [b.shape[1] for b in bs], evs, c,
                                                                                 rows, N, K, dev=dev, a_where=nv.VT_DEVICE),
                    dA_stream, dB, hC, blocks, mark_ready=mark_ready)
            elif shared_b:
                sharding.run_row_sharded(lambda a, b, c: host_call(a, b, c, nv.VT_HOST_AC_DEVICE_B), hA, dB, hC,
                                         B_source=hB)
            else:
                host_call(hA, hB, hC, nv.VT_HOST)

        def floor_step():
            # the same bytes over the same link as plain copies, both directions at once, no compute
            with torch.cuda.stream(copy_in):
                if hB is not None:
                    job.B.copy_(hB, non_blocking=True)
                job.A.copy_(hA, non_blocking=True)
            with torch.cuda.stream(copy_out):
                hC.copy_(job.C, non_blocking=True)

        def wall(fn, n):
            fn()
            barrier()
            t0 = time.perf_counter()
            for _ in range(n):
                fn()
            barrier()
            return ctx["max"]((time.perf_counter() - t0) / n)

        e2e_s = wall(e2e_step, e2e_steps)
        parity_host = job.check(hC)
        copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
        floor_s = wall(floor_step, e2e_steps)
        h2d = ctx["sum"](float((rows * K + (K * N if hB is not None else 0)) * job.elem_in))
        d2h = ctx["sum"](float(rows * N * job.elem_out))
        e2e = {"value": 2.0 * job.total_rows * N * K / e2e_s / 1e12, "unit": unit, "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h), "steps": e2e_steps, "ms_per_step": e2e_s * 1e3,
               "link_floor_ms": floor_s * 1e3, "over_link_floor": e2e_s / floor_s,
               "bytes": "whole job, all ranks; " + ("B crosses the host link on rank 0 only, in %d column blocks, and "
                                                     "reaches the other GPUs by NCCL broadcasts inside the timed "
                                                     "region; every rank computes and returns the columns of C a "
                                                     "block completes while later blocks arrive"
                                                     % len(blocks) if streamed else
                                                     "B crosses the host link on rank 0 only and reaches the other "
                                                     "GPUs by the NCCL broadcast inside the timed region"
                                                     if shared_b else "every rank copies the operands it uses"),
               "link_floor": "plain cudaMemcpyAsync of the same bytes on every rank at once, host->device and "
                             "device->host on two streams, no compute, wall clock, max over ranks"}

    parity = {"device_run": parity_device, "host_buffer_run": parity_host,
              "ok": bool(ctx["min"](1.0 if parity_device["ok"] and (parity_host is None or parity_host["ok"]) else 0.0) > 0.5),
              "ranks": world, "against": "exact product of the sampled rows in float64 on the GPU (int8: every bit; "
                                         "fp32: relative Frobenius error <= 1e-5)"}

    # ---- the weak-scaling figure beside the strong one: every rank the whole shape ----
    weak = None
    if world > 1 and args.scaling == "strong" and not job.replicas and not args.no_also:
        wjob = Job(ctx, args.workload, "weak", args.i8_variant, args.sgemm_variant)
        w_ms, _ = wjob.timed(steps, warm)
        weak = {"ms_per_step": w_ms, "value": wjob.value(w_ms), "unit": unit, "rows_per_gpu": wjob.rows,
                "parity_ok": bool(ctx["min"](1.0 if wjob.check(wjob.C)["ok"] else 0.0) > 0.5)}
        wjob.release()

    # ---- the other named workloads, each timed like the headline ----
    also = None
    if not args.no_also:
        also = {}
        # The short launches first, and a pause before each: right after a second at the power cap the GPU runs a
        # 20 us kernel half as fast again (640^3: 28 us in that position, 18.5 us on its own), which says nothing
        # about the kernel.
        for name, wl, variant in (("sgemm_256", "sgemm_256", nv.VT_SGEMM_AUTO),
                                  ("sgemm_640", "sgemm_640", nv.VT_SGEMM_AUTO),
                                  ("i8_64", "i8_64", 0),
                                  ("sgemm_skinny", "sgemm_skinny", nv.VT_SGEMM_AUTO),
                                  ("sgemm_8192", "sgemm_8192", nv.VT_SGEMM_AUTO),
                                  ("sgemm_8192_ffma", "sgemm_8192", nv.VT_SGEMM_TILE128),
                                  ("i8_batched", "i8_batched", 0)):
            if wl == args.workload and variant == args.sgemm_variant:
                continue
            time.sleep(0.25)
            j = Job(ctx, wl, "strong", 0, variant)
            a_ms, a_launches = j.timed(steps, warm)
            ok = bool(ctx["min"](1.0 if j.check(j.C)["ok"] else 0.0) > 0.5)
            roof = roofline_for(wl, j.kind, j.rows, j.N, j.K, a_ms, peaks, peaks_src, variant, nv)
            also[name] = {"metric": metric_of(wl)[0], "ms_per_step": a_ms, "value": j.value(a_ms), "unit": metric_of(wl)[1],
                          "rows_per_gpu": j.rows, "global_rows": int(j.total_rows), "launches": int(a_launches),
                          "steps": steps, "parity_ok": ok,
                          "sharding": "replicas (too few rows to shard); value is one replica's" if j.replicas else
                                      ("batch dealt over the ranks" if j.kind == "i8b" else "M rows per rank") if world > 1 else "single GPU",
                          "roofline": {k: roof[k] for k in ("bound", "achieved", "peak", "unit", "frac")}}
            if a_ms < 0.03:
                # launch-bound: the same 20 calls as one CUDA graph
                g_ms = j.graph_ms(steps)
                also[name]["graph_replay"] = {"ms_per_step": g_ms, "value": j.value(g_ms)}
            if j.kind == "f32":
                chosen = variant or nv.sgemm_auto_variant(j.rows, j.N, j.K, dev=ctx["dev"])
                also[name]["kernel"] = nv.SGEMM_VARIANT_NAMES.get(chosen, str(chosen))
            j.release()

    # ---- the same step back to back for about a second: NVML's clock and power readings lag a region of a
    # few milliseconds, so this is where the power cap shows; reported beside the timed region, not as it.  It
    # comes last: a second at full power warms the GPU, and nothing else is measured after it ----
    sustained = None
    if args.sustain_seconds > 0:
        reps = max(steps, min(200000, int(args.sustain_seconds * 1e3 / max(ms_per_step, 1e-3))))
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t_s0 = time.perf_counter()
        s0.record()
        for _ in range(reps):
            job.step()
        s1.record()
        barrier()
        t_s1 = time.perf_counter()
        sus_ms = ctx["max"](s0.elapsed_time(s1) / reps)
        nv.sync(dev, ctx["st"])
        if rank == 0:
            # the second half of the window: the readings have caught up with the load by then
            sustained = sampler.window(0.5 * (t_s0 + t_s1), t_s1) or {}
            sustained.update({"steps": reps, "ms_per_step": sus_ms, "seconds": t_s1 - t_s0})

    clocks = sampler.stop() if rank == 0 else None
    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0

    roof = roofline_for(args.workload, kind, rows, N, K, ms_per_step, peaks, peaks_src, args.sgemm_variant, nv)
    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling if world > 1 else "strong",
        "vs_baseline": None, "dtype": "f32" if kind == "f32" else "s8->s32", "data": "synthetic",
        "config": {"workload": args.workload, "M_per_gpu": rows, "N": N, "K": K, "global_M": global_rows,
                   "sharding": ("rows [r*M/g, (r+1)*M/g) of A and C per rank, B replicated: broadcast from rank 0 before "
                                "the timed region; no data-path collective") if world > 1 else "single GPU",
                   "comm_init_ms": comm_init_ms, "bcast_ms_warm": bcast_ms_warm,
                   "bcast": "comm_init_ms: process group + first 4-byte broadcast (communicator creation), wall clock; "
                            "bcast_ms_warm: one more broadcast of B on the warm communicator, CUDA events, max over ranks"
                            if world > 1 else None,
                   "l2": "working set per launch %.0f MiB > 126 MB L2; no flush between steps"
                         % ((rows * K * (1 if kind != "f32" else 4) + K * N * (1 if kind != "f32" else 4) + rows * N * 4) / 2**20),
                   "launch": "steps are enqueued back to back; the kernels are launched with programmatic stream "
                             "serialization (a step's set-up may overlap the end of the step before it; it touches "
                             "memory only after that step has completed)"},
        "clocks": clocks,
        "sustained": None if sustained is None else dict(
            sustained, value=value * ms_per_step / sustained["ms_per_step"], unit=unit,
            note="the same step repeated back to back after the timed region; clocks are NVML samples of the second "
                 "half of that window"),
        "e2e": e2e,
        "parity": parity,
        "gpu_launches": int(launches),
        "roofline": roof,
    }
    if weak is not None:
        line["weak"] = weak
    if also is not None:
        line["also"] = also
    if world == 1 and not args.no_cpu_baseline:
        arm = make_cpu_arm(args, kind if kind != "i8b" else "i8", M * batch if kind == "i8b" else M, N, K)
        rows_cpu = arm.size_sample(12.0)
        t = arm.run_rows(rows_cpu)
        line["cpu_baseline"] = {"value": arm.ops(rows_cpu) / t / 1e12, "unit": unit, "cores": arm.threads,
                                "kind": arm.kind_label, "sample": arm.describe(rows_cpu), "seconds": t}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


SHAPE_GRID = ((256, 256, 256), (512, 512, 512), (768, 768, 768), (1024, 1024, 1024), (2048, 2048, 2048), (256, 256, 8192),
              (512, 512, 8192), (1024, 256, 4096), (8192, 16, 8192), (8192, 64, 8192), (8192, 128, 8192), (8192, 256, 8192),
              (65536, 16, 1024), (4096, 32, 4096), (2048, 64, 2048), (16384, 128, 512), (16, 8192, 8192), (64, 8192, 8192),
              (128, 8192, 8192), (300, 8192, 8192), (384, 4096, 4096), (512, 8192, 8192), (1024, 8192, 1024), (128, 512, 512),
              (200, 300, 400), (2000, 200, 2000), (4096, 4096, 256), (4096, 4096, 64), (8192, 8192, 128), (128, 128, 65536),
              (1024, 64, 16384), (640, 640, 640), (1536, 1536, 1536), (3072, 512, 3072), (512, 3072, 3072), (896, 896, 896),
              (1000, 1000, 1000), (384, 384, 4096), (332, 776, 1112), (128, 128, 16384))


def run_shape_grid(shapes):
    """`--shape-grid`: every fp32 kernel variant of the library on a grid of shapes, beside the automatic choice and
    cuBLAS (`torch.matmul`, TF32 off) - the measurement behind the automatic choice in vt_sgemm.  Prints a
    markdown table; device-resident operands, CUDA events, 10 launches after 2 warm-up launches per cell."""
    import torch

    from veritac_b200 import _native as nv
    from veritac_b200 import build

    build.build()
    torch.backends.cuda.matmul.allow_tf32 = False
    names = {nv.VT_SGEMM_TILE128: "tile128", nv.VT_SGEMM_TILE64: "tile64", nv.VT_SGEMM_TILE32: "tile32",
             nv.VT_SGEMM_PIPE128: "pipe128", nv.VT_SGEMM_PIPE64X128: "pipe64x128", nv.VT_SGEMM_PIPE64: "pipe64",
             nv.VT_SGEMM_TF32X3: "tf32x3", nv.VT_SGEMM_PANEL_TF32X3: "panel", nv.VT_SGEMM_TALL_TF32X3: "tall"}
    st = nv.torch_stream()

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 10

    print("| M x N x K | automatic | chosen | best single variant | automatic / best | cuBLAS | automatic / cuBLAS | "
          + " | ".join(names.values()) + " |")
    print("|---|---|---|---|---|---|---|" + "---|" * len(names))
    slower = 0
    ratios = []
    for (m, n, k) in shapes:
        A = torch.rand((m, k), device="cuda") * 2 - 1
        B = torch.rand((k, n), device="cuda") * 2 - 1
        C = torch.empty((m, n), device="cuda")
        cells = {}
        for variant in names:
            if variant == nv.VT_SGEMM_PANEL_TF32X3 and m > 512:
                continue
            try:
                cells[variant] = timed(lambda: nv.sgemm(A, B, C, m, n, k, variant=variant, where=nv.VT_DEVICE, stream=st))
                nv.sync(0, st)
            except nv.NativeError:
                pass
        auto = timed(lambda: nv.sgemm(A, B, C, m, n, k, where=nv.VT_DEVICE, stream=st))
        nv.sync(0, st)
        lib = timed(lambda: torch.matmul(A, B, out=C))
        best = min(cells, key=cells.get)
        slower += auto > 1.03 * lib
        ratios.append((auto / cells[best], auto / lib))
        chosen = nv.SGEMM_VARIANT_NAMES.get(nv.sgemm_auto_variant(m, n, k), "?")
        print("| %d x %d x %d | %.4f ms | %s | %s %.4f | %.2f | %.4f | %.2f | "
              % (m, n, k, auto, chosen, names[best], cells[best], auto / cells[best], lib, auto / lib)
              + " | ".join("%.4f" % cells[v] if v in cells else "-" for v in names) + " |", flush=True)
    print("\nautomatic choice slower than cuBLAS by more than 3 %% on %d of %d shapes" % (slower, len(shapes)))
    if ratios:
        gm = lambda xs: math.exp(sum(math.log(x) for x in xs) / len(xs))
        print("geometric mean of automatic / best single variant %.3f, of automatic / cuBLAS %.3f"
              % (gm([r[0] for r in ratios]), gm([r[1] for r in ratios])))
    return 0


def random_mid_shapes(seed, count):
    """Seeded mid-sized fp32 shapes for `--shape-grid --random-shapes`: cubes of 160 to 1600, long-K products, wide and
    tall ones; N and K multiples of 4."""
    import numpy as np
    rng = np.random.default_rng(seed)
    shapes = []
    for _ in range(count):
        kind = rng.integers(0, 4)
        if kind == 0:
            m = n = k = 4 * int(rng.integers(40, 400))
        elif kind == 1:
            m, n, k = 4 * int(rng.integers(20, 300)), 4 * int(rng.integers(20, 300)), 4 * int(rng.integers(100, 4000))
        elif kind == 2:
            m, n, k = 4 * int(rng.integers(50, 800)), 4 * int(rng.integers(10, 200)), 4 * int(rng.integers(50, 1000))
        else:
            m, n, k = 4 * int(rng.integers(10, 600)), 4 * int(rng.integers(50, 800)), 4 * int(rng.integers(50, 1000))
        shapes.append((m, n, k))
    return shapes


def metric_of(workload):
    kind, M, N, K, batch = WORKLOADS[workload]
    if kind == "f32":
        return "fp32 GEMM TFLOPS at %dx%dx%d" % (M, N, K), "TFLOPS"
    if kind == "i8b":
        return "exact int8->int32 batched B-reuse GEMM TOPS (%d x %dx%dx%d)" % (batch, M, N, K), "TOPS"
    return ("exact int8->int32 GEMM TOPS at %d^3" % M if M == N == K else
            "exact int8->int32 GEMM TOPS at %dx%dx%d" % (M, N, K)), "TOPS"


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("b200", "reference"), default="b200")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="i8_8192")
    ap.add_argument("--scaling", choices=("weak", "strong"), default="strong",
                    help="strong: the shape's rows are split over the GPUs; weak: every GPU gets the full shape")
    ap.add_argument("--i8-variant", type=int, default=0, help="VT_I8_* kernel variant (0 = the library's choice)")
    ap.add_argument("--sgemm-variant", type=int, default=0, help="VT_SGEMM_* kernel variant (0 = the library's choice)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sustain-seconds", type=float, default=1.0,
                    help="after the timed region, repeat the step for about this long and report its rate and the "
                         "clocks NVML shows under that load (0 = skip)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-also", action="store_true", help="skip the other workloads and the weak figure")
    ap.add_argument("--shape-grid", nargs="*", metavar="MxNxK", default=None,
                    help="instead of a bench line: time every fp32 kernel variant, the automatic choice and cuBLAS on "
                         "these shapes (no shapes: the built-in grid of 40) and print a markdown table")
    ap.add_argument("--random-shapes", metavar="SEED:COUNT", default=None,
                    help="with --shape-grid: COUNT seeded random mid-sized shapes instead of the built-in grid")
    args = ap.parse_args()
    if args.shape_grid is not None:
        if args.random_shapes:
            seed, count = (int(x) for x in args.random_shapes.split(":"))
            return run_shape_grid(random_mid_shapes(seed, count))
        return run_shape_grid([tuple(int(x) for x in a.lower().split("x")) for a in args.shape_grid] or list(SHAPE_GRID))
    kind, M, N, K, batch = WORKLOADS[args.workload]
    metric, unit = metric_of(args.workload)
    if args.impl == "reference":
        return run_reference_arm(args, "i8" if kind == "i8b" else kind, M * batch if kind == "i8b" else M, N, K,
                                 metric, unit)
    return run_gpu_arm(args, kind, M, N, K, batch, metric, unit)


if __name__ == "__main__":
    sys.exit(main())
