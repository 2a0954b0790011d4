"""Headline numbers of one simulated step.
Reference role: ``src/dataflow_sim/workloads/summary.py:15-59`` (``compute_summary``)."""
from __future__ import annotations

from ..schema import EventLog, TaskChain


def compute_summary(chain: TaskChain, log: EventLog, program=None) -> dict:
    """Makespan, tokens/s, model TFLOP/s, memory peaks, recompute share, idle share and lane busy times.
    ``program``: the ``WorkloadProgram`` the chain came from (for tokens, FLOPs and phases), optional."""
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
           "stall_us": float(sum(log.stalls.values()))}
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
                   recompute_pct=100.0 * by_phase.get("recompute", 0.0) / busy if busy else 0.0, busy_by_phase_us=by_phase)
    return out


def _moved(chain: TaskChain, log: EventLog, direction: str) -> int:
    sizes = chain.sizes()
    return int(sum(sizes.get(iv.task_id.split(":", 1)[-1], 0) for iv in log.transfer_intervals(direction)))
