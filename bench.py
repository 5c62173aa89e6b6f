#!/usr/bin/env python3
"""Benchmark of the B200 GEMM back end on the reference's headline workload.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One JSON line on stdout (rank 0).  A *step* is one pass of the hot path over one batch of synthetic
input: one GEMM of the named shape per GPU.  Default workload: exact int8 x int8 -> int32 GEMM,
M = N = K = 8192 per GPU (BASELINE.json configs[2]); with N GPUs every rank owns 8192 rows of a
(8192*N) x 8192 A and C (M-row sharding, weak scaling) and B is broadcast once from rank 0 over NCCL
before timing.  There is no data-path collective.

  value      whole-job throughput, operands resident in HBM, CUDA-event time on the launching
             stream, max over ranks
  e2e        same metric through the C ABI with pinned HOST buffers: host->device copies of A and B
             and the device->host copy of C are inside the timed region of every step
  roofline   achieved = algorithmic ops (or bytes) per launch / average launch duration of the
             timed region; peak from MEASURED_PEAKS.json (fallback stated if absent)
  cpu_baseline  the oracle's OpenMP C restatement of the reference's CPU arithmetic, timed on this
             host's cores on a bounded sample of the same workload (N = 1 only)

`--impl reference` times that CPU restatement alone, with every host thread, on bounded samples of
the same workload, and prints the same line shape with "impl": "reference".
"""
from __future__ import annotations

import argparse
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

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/; None until a capture exists for the workload.
NCU_TRAFFIC_BYTES = {"sgemm_skinny": 273.9e6, "sgemm_panel_128": 282.9e6, "sgemm_tall_16": 275.8e6, "i8_8192": 590.1e6, "i8_batched_32": 654.4e6, "i8_batched": 8 * 654.4e6}

WORKLOADS = {
    # name: (kind, M, N, K, batch)
    "i8_8192": ("i8", 8192, 8192, 8192, 1),
    "i8_64": ("i8", 64, 64, 64, 1),
    "i8_batched": ("i8b", 1024, 4096, 4096, 256),
    "i8_batched_32": ("i8b", 1024, 4096, 4096, 32),      # one GPU's share of config 4 on 8 GPUs
    "sgemm_8192": ("f32", 8192, 8192, 8192, 1),
    "sgemm_256": ("f32", 256, 256, 256, 1),
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
        "warmup": warm, "ms_per_step": total / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32" if kind == "f32" else "s8->s32", "data": "synthetic",
        "config": {"workload": args.workload, "M": M, "N": N, "K": K,
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
def run_gpu_arm(args, kind, M, N, K, batch, metric, unit):
    import numpy as np
    import torch
    import torch.distributed as dist

    from veritac_b200 import _native as nv
    from veritac_b200 import build, sharding

    build.build()
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
    rows = M * batch                     # rows this rank owns (weak scaling: per-GPU work is fixed)
    if args.scaling == "strong":
        r0, r1 = sharding.row_shard(M * batch, world, rank, align=M if kind == "i8b" else 16)
        rows = r1 - r0
    gen = torch.Generator(device="cuda").manual_seed(20260917 + rank)
    st = nv.torch_stream()

    # Operands: A differs per rank (its own row block); B comes from rank 0 by one broadcast.
    if kind == "f32":
        A = torch.rand((rows, K), device="cuda", generator=gen) * 2 - 1
        B = torch.rand((K, N), device="cuda", generator=gen) * 2 - 1
        C = torch.zeros((rows, N), device="cuda")
        elem_in, elem_out = 4, 4
    else:
        A = torch.randint(-128, 128, (rows, K), dtype=torch.int8, device="cuda", generator=gen)
        B = torch.randint(-128, 128, (K, N), dtype=torch.int8, device="cuda", generator=gen)
        C = torch.empty((rows, N), dtype=torch.int32, device="cuda")
        elem_in, elem_out = 1, 4
    t_b0 = time.perf_counter()
    sharding.replicate_from_rank0(B)
    torch.cuda.synchronize()
    bcast_ms = (time.perf_counter() - t_b0) * 1e3

    def step():
        if kind == "f32":
            nv.sgemm(A, B, C, rows, N, K, dev=dev, variant=args.sgemm_variant, where=nv.VT_DEVICE, stream=st)
        elif kind == "i8b":
            nv.i8gemm_shared_b(A, B, C, rows // M, M, N, K, dev=dev, acc_rows=16, where=nv.VT_DEVICE, stream=st)
        else:
            nv.i8gemm(A, B, C, rows, N, K, dev=dev, variant=args.i8_variant, where=nv.VT_DEVICE, stream=st)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warm):
        step()
    nv.sync(dev, st)
    barrier()
    try:
        gpu_uuid = str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        gpu_uuid = None
    sampler = ClockSampler(local, gpu_uuid)
    if rank == 0:
        sampler.start()
        time.sleep(0.05)
    launches0 = nv.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.mark_begin()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    sampler.mark_end()
    elapsed_ms = e0.elapsed_time(e1)
    launches = nv.launch_count() - launches0
    nv.sync(dev, st)
    if world > 1:
        t = torch.tensor([elapsed_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
        tot = torch.tensor([float(rows)], device="cuda", dtype=torch.float64)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        total_rows = float(tot.item())
    else:
        total_rows = float(rows)
    ms_per_step = elapsed_ms / steps

    # ---- the same step back to back for about a second: NVML's clock and power readings lag a region of a
    # few milliseconds, so this is where the power cap shows; reported beside the timed region, not as it ----
    sustained = None
    if args.sustain_seconds > 0:
        reps = max(steps, min(200000, int(args.sustain_seconds * 1e3 / max(ms_per_step, 1e-3))))
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t_s0 = time.perf_counter()
        s0.record()
        for _ in range(reps):
            step()
        s1.record()
        barrier()
        t_s1 = time.perf_counter()
        sus_ms = s0.elapsed_time(s1) / reps
        nv.sync(dev, st)
        if world > 1:
            t = torch.tensor([sus_ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sus_ms = float(t.item())
        if rank == 0:
            # the second half of the window: the readings have caught up with the load by then
            sustained = sampler.window(0.5 * (t_s0 + t_s1), t_s1) or {}
            sustained.update({"steps": reps, "ms_per_step": sus_ms, "seconds": t_s1 - t_s0})
    clocks = sampler.stop() if rank == 0 else None
    ops_per_step_job = 2.0 * total_rows * N * K
    value = ops_per_step_job / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the C ABI with pinned host buffers (every rank, its own block) ----
    e2e_steps = max(2, min(steps, 5))
    hA = torch.empty((rows, K), dtype=A.dtype).pin_memory()
    hB = torch.empty((K, N), dtype=B.dtype).pin_memory()
    hC = torch.empty((rows, N), dtype=C.dtype).pin_memory()
    hA.copy_(A)
    hB.copy_(B)

    def e2e_step():
        if kind == "f32":
            nv.sgemm(hA, hB, hC, rows, N, K, dev=dev, where=nv.VT_HOST)
        elif kind == "i8b":
            nv.i8gemm_shared_b(hA, hB, hC, rows // M, M, N, K, dev=dev, acc_rows=16, where=nv.VT_HOST)
        else:
            nv.i8gemm(hA, hB, hC, rows, N, K, dev=dev, where=nv.VT_HOST)

    if args.no_e2e:
        e2e_steps = 0
        e2e_s = None
    else:
        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1 and e2e_s:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = ops_per_step_job / e2e_s / 1e12 if e2e_s else None
    e2e_ok = bool(torch.equal(hC[:64].cuda(), C[:64])) if kind != "f32" and not args.no_e2e else None
    h2d = (rows * K + K * N) * elem_in
    d2h = rows * N * elem_out

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0

    # ---- roofline of the dominant kernel (this rank's launch) ----
    launch_ms = ms_per_step
    ops_per_launch = 2.0 * rows * N * K
    algo_bytes = (K * N + rows * K + rows * N) * 4.0
    tf32x3_peak = peaks["bf16_tflops"] / 2.0 / 3.0       # three TF32 MMAs per fp32 product; TF32 at half the bf16 rate
    panel = args.workload in ("sgemm_skinny", "sgemm_panel_64", "sgemm_panel_128", "sgemm_tall_16")
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
        tensor_path = args.sgemm_variant == nv.VT_SGEMM_TF32X3 or (
            args.sgemm_variant == nv.VT_SGEMM_AUTO and rows >= 256 and N >= 256 and K >= 256
            and float(rows) * N * K >= 5.0e8 and N % 4 == 0 and K % 4 == 0)
        if tensor_path:
            # three TF32 MMAs per fp32 product; TF32 issues at half the bf16 rate
            peak = peaks["bf16_tflops"] / 2.0 / 3.0
            roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
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
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_source": "2 x %s bf16_tflops (kind::i8 issues at twice the bf16 rate)" % peaks_src,
                "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS}
    roof["traffic"] = NCU_TRAFFIC_BYTES.get(args.workload)
    roof["launch_ms"] = launch_ms

    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": "f32" if kind == "f32" else "s8->s32", "data": "synthetic",
        "config": {"workload": args.workload, "M_per_gpu": rows, "N": N, "K": K, "global_M": int(total_rows),
                   "sharding": "M rows per rank, B broadcast once from rank 0 (%.2f ms, outside the timed region), "
                               "no data-path collective" % bcast_ms if world > 1 else "single GPU",
                   "l2": "working set per launch %.0f MiB > 126 MB L2; no flush between steps"
                         % ((rows * K * elem_in + K * N * elem_in + rows * N * elem_out) / 2**20),
                   "launch": "steps are enqueued back to back; the kernels are launched with programmatic stream "
                             "serialization (a step's set-up may overlap the end of the step before it; it touches "
                             "memory only after that step has completed)"},
        "clocks": clocks,
        "sustained": None if sustained is None else dict(
            sustained, value=ops_per_step_job / (sustained["ms_per_step"] * 1e-3) / 1e12, unit=unit,
            note="the same step repeated back to back after the timed region; clocks are NVML samples of the second "
                 "half of that window"),
        "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "steps": e2e_steps, "ms_per_step": e2e_s * 1e3 if e2e_s else None, "matches_device_run": e2e_ok},
        "gpu_launches": int(launches),
        "roofline": roof,
    }
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


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("b200", "reference"), default="b200")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="i8_8192")
    ap.add_argument("--scaling", choices=("weak", "strong"), default="weak",
                    help="weak: every GPU gets the full shape; strong: the shape's rows are split over the GPUs")
    ap.add_argument("--i8-variant", type=int, default=0, help="VT_I8_* kernel variant (0 = the library's choice)")
    ap.add_argument("--sgemm-variant", type=int, default=0, help="VT_SGEMM_* kernel variant (0 = the library's choice)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sustain-seconds", type=float, default=1.0,
                    help="after the timed region, repeat the step for about this long and report its rate and the "
                         "clocks NVML shows under that load (0 = skip)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    args = ap.parse_args()
    kind, M, N, K, batch = WORKLOADS[args.workload]
    if kind == "f32":
        metric, unit = "fp32 GEMM TFLOPS at %dx%dx%d" % (M, N, K), "TFLOPS"
    elif kind == "i8b":
        metric, unit = "exact int8->int32 batched B-reuse GEMM TOPS (%d x %dx%dx%d)" % (batch, M, N, K), "TOPS"
    else:
        metric, unit = "exact int8->int32 GEMM TOPS at %d^3" % M if M == N == K else \
            "exact int8->int32 GEMM TOPS at %dx%dx%d" % (M, N, K), "TOPS"
    if args.impl == "reference":
        return run_reference_arm(args, "i8" if kind == "i8b" else kind, M * batch if kind == "i8b" else M, N, K,
                                 metric, unit)
    return run_gpu_arm(args, kind, M, N, K, batch, metric, unit)


if __name__ == "__main__":
    sys.exit(main())
