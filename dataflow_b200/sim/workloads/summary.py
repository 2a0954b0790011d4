"""Headline numbers of one simulated step.
Reference role: ``src/dataflow_sim/workloads/summary.py:15-59`` (``compute_summary``)."""
from __future__ import annotations

from ..schema import EventLog, TaskChain


def compute_summary(chain: TaskChain, log: EventLog, program=None, hw=None) -> dict:
    """Makespan, tokens/s, model TFLOP/s, memory peaks, recompute share, idle share and lane busy times.
    ``program``: the ``WorkloadProgram`` the chain came from (for tokens, FLOPs and phases), optional.  With ``hw`` (the
    ``HardwareSpec`` the chain was priced on) also: where the compute time goes by kind of op (tensor-core matmuls,
    attention, memory-bound element-wise work, fabric collectives), model FLOP utilisation against the hardware's peak, the
    ten most expensive ops, and the lanes' utilisation."""
    makespan = float(log.makespan)
    compute = log.compute_intervals()
    busy = sum(iv.end - iv.start for iv in compute)
    lanes = {d: sum(iv.end - iv.start for iv in log.transfer_intervals(d)) for d in ("from_slow", "to_slow")}
    out = {"makespan_us": makespan, "compute_busy_us": busy, "idle_us": max(makespan - busy, 0.0),
           "idle_pct": 100.0 * max(makespan - busy, 0.0) / makespan if makespan else 0.0,
           "from_slow_busy_us": lanes["from_slow"], "to_slow_busy_us": lanes["to_slow"],
           "from_slow_bytes": _moved(chain, log, "from_slow"), "to_slow_bytes": _moved(chain, log, "to_slow"),
           "peak_fast_bytes": int(log.peak_fast_memory_bytes), "peak_backing_bytes": int(log.peak_backing_memory_bytes),
           "fast_capacity_bytes": chain.fast_memory_capacity, "stalled_tasks": len(log.stalls),
           "stall_us": float(sum(log.stalls.values())),
           "from_slow_util_pct": 100.0 * lanes["from_slow"] / makespan if makespan else 0.0,
           "to_slow_util_pct": 100.0 * lanes["to_slow"] / makespan if makespan else 0.0,
           "peak_fast_memory_gb": log.peak_fast_memory_bytes / 1e9,
           "worst_stalls": [{"task": k, "us": float(v)} for k, v in sorted(log.stalls.items(), key=lambda kv: -kv[1])[:5]]}
    if program is not None:
        tokens = int(program.metadata.get("tokens_per_step", 0))
        flops = sum(op.flops for t in program.tasks for op in t.cost.ops)
        phase = {t.id: t.phase for t in program.tasks}
        by_phase: dict[str, float] = {}
        for iv in compute:
            by_phase[phase.get(iv.task_id, "other")] = by_phase.get(phase.get(iv.task_id, "other"), 0.0) + (iv.end - iv.start)
        rec_flops = sum(op.flops for t in program.tasks if t.phase == "recompute" for op in t.cost.ops)
        out.update(tokens=tokens, tokens_per_s=tokens / makespan * 1e6 if makespan else 0.0,
                   total_flops=flops, tflops=flops / makespan / 1e6 if makespan else 0.0,
                   model_tflops=(flops - rec_flops) / makespan / 1e6 if makespan else 0.0,
                   recompute_pct=100.0 * by_phase.get("recompute", 0.0) / busy if busy else 0.0, busy_by_phase_us=by_phase,
                   primary_unit="tokens", primary_count=tokens, primary_rate_per_second=tokens / makespan * 1e6 if makespan else 0.0,
                   flops_by_phase={ph: float(sum(op.flops for t in program.tasks if (t.phase or "other") == ph for op in t.cost.ops))
                                   for ph in sorted({t.phase or "other" for t in program.tasks})})
        if hw is not None:
            from .schema import resolve_subop
            by_kind: dict[str, float] = {}
            ops: dict[str, list] = {}
            for t in program.tasks:
                for op in t.cost.ops:
                    us = resolve_subop(op, hw)
                    by_kind[op.kind] = by_kind.get(op.kind, 0.0) + us
                    # the same op of every layer and round under one name: drop the layer-free prefix the tracer gives
                    rec = ops.setdefault(op.name, [0.0, 0.0, 0, op.kind])
                    rec[0] += us
                    rec[1] += op.flops
                    rec[2] += 1
            total = sum(by_kind.values()) or 1.0
            peak = hw.tflops(program.metadata.get("compute_dtype", "bf16"))
            out.update(compute_us_by_kind=by_kind, compute_pct_by_kind={k: 100.0 * v / total for k, v in by_kind.items()},
                       hardware_peak_tflops=peak, mfu_pct=100.0 * out["model_tflops"] / peak if peak else 0.0,
                       top_ops=[{"name": n, "kind": r[3], "us": r[0], "flops": r[1], "calls": r[2], "pct_of_compute": 100.0 * r[0] / total}
                                for n, r in sorted(ops.items(), key=lambda kv: -kv[1][0])[:10]])
    return out


def _moved(chain: TaskChain, log: EventLog, direction: str) -> int:
    sizes = chain.sizes()
    return int(sum(sizes.get(iv.task_id.split(":", 1)[-1], 0) for iv in log.transfer_intervals(direction)))
