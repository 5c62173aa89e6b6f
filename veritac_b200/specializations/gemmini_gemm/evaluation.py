"""Controls for a candidate Gemmini stream, with measured B200 time beside the modeled traffic.

Counterpart of the reference's specializations/gemmini_gemm/evaluation.py (`objective` :10-12,
`compare_controls` :15-51).  The reference scores a candidate against the baseline stream and every
batched B-reuse stream that fits the plan's accumulator, by *modeled* bytes only, and gates each
stream on its Lean program checker (out of reach here: that checker stays with the reference).
`measure_controls` keeps the same proposals, the same modeled objective and the same result keys,
gates each stream on the symbolic replay that `run_commands` uses (every rule of the reference
interpreter), and fills the reference's always-None `hardware_latency` with what the stream's
schedule costs on the GPU: device-resident time of the GEMM launched with that stream's tile order.
"""
from __future__ import annotations

from . import backend as g
from .lowering import command_hash, gen_batched_reuse_b


DEFAULT_INTERPRET_MACS_LIMIT = 4_000_000


def interpret_commands(plan, commands, interpret_macs_limit=DEFAULT_INTERPRET_MACS_LIMIT):
    """Exact interpretation of a candidate stream on the deterministic inputs, as the reference's search
    controller does for every natively accepted candidate (blind_search.py:959-976, bound :65): the same
    result dictionary (`ran`, `matches_reference`, `error` / `reason`), with the stream executed on the
    GPU by `run_commands` and compared with `scalar_matmul`.  Diagnostic only, like the original: it never
    stands in for the plan checker."""
    macs = plan["m"] * plan["n"] * plan["k"]
    if macs > interpret_macs_limit:
        return {"ran": False,
                "reason": "skipped: %d modeled MACs exceed the interpretation bound %d" % (macs, interpret_macs_limit)}
    A, B = g.deterministic_inputs(plan["m"], plan["n"], plan["k"], 0)
    try:
        C, _stats = g.run_commands(commands, plan, A, B)
    except g.GemminiError as exc:
        return {"ran": True, "matches_reference": False, "error": str(exc)}
    return {"ran": True, "matches_reference": C == g.scalar_matmul(A, B, plan["m"], plan["n"], plan["k"])}


def objective(commands):
    counts = g.modeled_counts(commands)
    return (counts["dma_in_elems_int8"], counts["instructions"])


def _replay(plan, commands):
    """(raster, live row tiles) of a stream that computes the plan's full GEMM; raises GemminiError."""
    replay = g._Replay(plan)
    for c in commands:
        replay.step(c)
    replay.finish()
    raster = g._plain_gemm_raster(replay.tiles, plan["m"], plan["n"], plan["k"])
    if raster is None:
        raise g.GemminiError("stream does not compute the plan's full GEMM")
    live = replay.max_acc_base // g.DIM + 1
    if raster == "reuse_b" and live < plan["m"] // g.DIM:
        raster = "batched"
    return raster, live


def measure_controls(plan, commands, A, B, *, repeats=20):
    """Score `commands` against the baseline and every batched B-reuse control of `plan`.

    A and B are int8 numpy arrays (m*k and k*n).  ValueError if the plan is invalid, the candidate
    stream is refused by the replay, or no control is admissible — as in the reference.  Every
    admissible stream is executed; `bit_exact` says all of them produced the same C.
    """
    import numpy as np
    import torch

    from ... import _native as nv

    ok, why = g.validate_plan(plan)
    if not ok:
        raise ValueError(why)
    accepted, why, _ = g.gemmini_check(plan)
    if not accepted:
        raise ValueError("candidate failed independent validation: " + why)
    try:
        cand_raster, cand_live = _replay(plan, commands)
    except g.GemminiError as exc:
        raise ValueError("candidate failed independent validation: %s" % exc) from exc
    m, n, k = plan["m"], plan["n"], plan["k"]
    dA = torch.from_numpy(np.ascontiguousarray(A, dtype=np.int8).reshape(m, k)).cuda()
    dB = torch.from_numpy(np.ascontiguousarray(B, dtype=np.int8).reshape(k, n)).cuda()
    stream = nv.torch_stream()
    dev = torch.cuda.current_device()
    codes = {"baseline": nv.VT_RASTER_BASELINE, "reuse_b": nv.VT_RASTER_REUSE_B, "batched": nv.VT_RASTER_BATCHED}

    def timed(raster, live):
        out = torch.full((m, n), -2**31, dtype=torch.int32, device="cuda")
        call = lambda: nv.i8gemm(dA, dB, out, m, n, k, dev=dev, raster=codes[raster],  # noqa: E731
                                 batch_rows=max(1, min(64, live)), where=nv.VT_DEVICE, stream=stream)
        call()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(repeats):
            call()
        e1.record()
        nv.sync(dev, stream)
        return e0.elapsed_time(e1) / repeats, out

    proposals = [("baseline", g.gen_commands(plan))]
    for batch in range(1, min(m // 16, plan["accumulator_rows"] // 16) + 1):
        proposals.append((f"existing_batched_b_{batch}", gen_batched_reuse_b(plan, batch)))
    controls, results = [], []
    for name, program in proposals:
        entry = {"name": name, "counts": g.modeled_counts(program), "objective": list(objective(program)),
                 "command_sha256": command_hash(program)}
        try:
            raster, live = _replay(plan, program)
            entry.update(native_accepted=True, reason="replayed")
            entry["gpu_time_ms"], out = timed(raster, live)
            results.append(out)
        except g.GemminiError as exc:
            entry.update(native_accepted=False, reason=str(exc), gpu_time_ms=None)
        controls.append(entry)
    admissible = [c for c in controls if c["native_accepted"]]
    if not admissible:
        raise ValueError("no validated control")
    cand_ms, cand_out = timed(cand_raster, cand_live)
    best = min(admissible, key=lambda c: c["objective"])
    counts = g.modeled_counts(commands)
    baseline = next(c for c in controls if c["name"] == "baseline")
    digest = command_hash(commands)
    return {
        "scope": "replay-validated modeled traffic with measured B200 time; no Lean program certificate",
        "counts": counts, "objective": list(objective(commands)), "controls": controls,
        "best_existing_control": best["name"],
        "input_reduction_vs_baseline": 1 - counts["dma_in_elems_int8"] / baseline["counts"]["dma_in_elems_int8"],
        "input_reduction_vs_best_existing": 1 - counts["dma_in_elems_int8"] / best["counts"]["dma_in_elems_int8"],
        "beats_best_existing_objective": list(objective(commands)) < best["objective"],
        "exact_matches": [c["name"] for c in admissible if c["command_sha256"] == digest],
        "fewer_a_loads_than_existing_controls": counts["mvin_A"] < min(c["counts"]["mvin_A"] for c in admissible),
        "novelty": "requires manual mechanism review; a distinct hash is insufficient",
        "hardware_latency": {"unit": "ms", "device": torch.cuda.get_device_name(dev), "candidate": cand_ms,
                             "fastest_control": min(admissible, key=lambda c: c["gpu_time_ms"])["name"]},
        "bit_exact": all(bool(torch.equal(cand_out, r)) for r in results),
    }
