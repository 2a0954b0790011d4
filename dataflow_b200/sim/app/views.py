"""Panel data of the simulator's front end, computed from a planned chain and its event log.

Pure functions, so that what the page shows can be tested without a browser:

    plan_table            the annotated plan, one row per task: what it reads and writes, what leaves and arrives after it
    residency_spans       for every object, the time intervals during which it holds fast memory (from the event stream)
    memory_by_type        fast memory over time split by object type, sampled for a stacked-area chart
    resident_at           who is in fast memory at a given time, largest first (the event scrubber)
    stall_rows            the stall report as rows: who waited, for what, how long; lane use
    reference_rows        the first-touch tape: in which order and when the chain first needs each object
    candidate_rows        the planner's own account of its search (PressureFit and Lookahead keep one)

Reference role: the data behind ``src/dataflow_sim/ui/src/components/{AnnotatedPlanPanel,MemoryBreakdown,MemoryTimelinePanel,
EventControls,PolicyDiagnosticsPanel,ReferenceStream}.tsx``.
"""
from __future__ import annotations

import bisect
from typing import Any

from ..reference_stream import compute_reference_stream, stall_free_starts
from ..schema import EventLog, TaskChain
from ..stall_report import build_stall_report


def plan_table(planned: TaskChain, log: EventLog | None = None) -> list[dict[str, Any]]:
    when = {iv.task_id: (iv.start, iv.end) for iv in log.task_intervals if iv.track == "compute"} if log else {}
    rows = []
    for i, t in enumerate(planned.tasks):
        s, e = when.get(t.id, (None, None))
        rows.append({"index": i, "task": t.id, "runtime_us": t.runtime, "start_us": s, "end_us": e,
                     "stall_us": (log.stalls.get(t.id, 0.0) if log else 0.0),
                     "inputs": list(t.inputs), "outputs": [o.id for o in t.outputs], "mutates": list(t.mutates_inputs),
                     "workspace_bytes": t.workspace_bytes, "releases": list(t.releases_after),
                     "offloads": [x.obj_id for x in t.offload_after], "prefetches": [x.obj_id for x in t.prefetch_after]})
    return rows


def residency_spans(planned: TaskChain, log: EventLog) -> dict[str, list[list[float]]]:
    """``{object: [[from, to], ...]}`` in microseconds.  Needs a log recorded with ``snapshots=True``."""
    if not log.events:
        raise ValueError("the event log has no events: simulate with snapshots=True")
    outputs = {t.id: [o.id for o in t.outputs if o.location == "fast"] for t in planned.tasks}
    open_at: dict[str, float] = {o.id: 0.0 for o in planned.initial_memory if o.location == "fast"}
    spans: dict[str, list[list[float]]] = {}

    def close(o: str, t: float) -> None:
        if o in open_at:
            spans.setdefault(o, []).append([open_at.pop(o), t])

    for ev in log.events:
        if ev.kind == "task_start":
            for o in outputs.get(ev.task_id or "", ()):
                open_at.setdefault(o, ev.t)
        elif ev.kind == "release":
            for o in ev.object_ids:
                close(o, ev.t)
        elif ev.kind == "transfer_start" and ev.transfer_direction == "from_slow":
            open_at.setdefault(ev.transfer_obj or "", ev.t)
        elif ev.kind == "transfer_end" and ev.transfer_direction == "to_slow":
            close(ev.transfer_obj or "", ev.t)
    end = log.makespan
    for o in list(open_at):
        close(o, max(end, open_at[o]))
    return spans


def memory_by_type(planned: TaskChain, log: EventLog, points: int = 240) -> dict[str, Any]:
    sizes = planned.sizes()
    types = {o.id: o.type for o in planned.initial_memory}
    for t in planned.tasks:
        for o in t.outputs:
            types[o.id] = o.type
    spans = residency_spans(planned, log)
    end = max(log.makespan, 1e-9)
    ts = [end * k / (points - 1) for k in range(points)]
    names = sorted({types.get(o, "other") for o in spans})
    series = {n: [0.0] * points for n in names}
    for o, ivs in spans.items():
        col = series[types.get(o, "other")]
        sz = sizes.get(o, 0)
        for a, b in ivs:
            lo = bisect.bisect_left(ts, a)
            hi = bisect.bisect_left(ts, b)           # resident on [a, b)
            for k in range(lo, hi):
                col[k] += sz
    return {"t_us": ts, "types": names, "bytes": series, "capacity_bytes": planned.fast_memory_capacity}


def resident_at(planned: TaskChain, log: EventLog, t_us: float, limit: int = 40) -> dict[str, Any]:
    sizes = planned.sizes()
    types = {o.id: o.type for o in planned.initial_memory}
    for t in planned.tasks:
        for o in t.outputs:
            types[o.id] = o.type
    here = [(sizes.get(o, 0), o) for o, ivs in residency_spans(planned, log).items() if any(a <= t_us < b for a, b in ivs)]
    here.sort(reverse=True)
    running = next((iv.task_id for iv in log.task_intervals if iv.track == "compute" and iv.start <= t_us < iv.end), None)
    moving = [iv.task_id for iv in log.task_intervals if iv.track != "compute" and iv.start <= t_us < iv.end]
    return {"t_us": t_us, "running": running, "moving": moving, "fast_bytes": sum(s for s, _ in here), "count": len(here),
            "objects": [{"id": o, "bytes": s, "type": types.get(o, "other")} for s, o in here[:limit]]}


def stall_rows(planned: TaskChain, log: EventLog, limit: int = 25) -> dict[str, Any]:
    rep = build_stall_report(planned, log)
    return {"stall_us": rep.stall_us, "stall_fraction": rep.stall_fraction, "by_object_type": dict(rep.by_object_type),
            "lanes": {k: {"transfers": v.transfers, "busy_us": v.busy_us, "busy_fraction": v.busy_fraction, "backlog_us": v.backlog_us}
                      for k, v in rep.lanes.items()},
            "stalls": [{"task": s.task_id, "index": s.index, "waited_us": s.stall_us, "inputs": list(s.waited_inputs),
                        "capacity": s.waited_capacity, "blocking_object": s.blocking_object} for s in rep.top(limit)],
            "text": rep.format(limit)}


def reference_rows(planned: TaskChain, limit: int = 400) -> list[dict[str, Any]]:
    sizes = planned.sizes()
    refs = compute_reference_stream(planned.tasks, stall_free_starts(planned.tasks))
    return [{"object": r.obj_id, "first_touch_us": r.ref_t, "task": r.ref_task, "bytes": sizes.get(r.obj_id, 0)} for r in refs[:limit]]


def candidate_rows(result) -> dict[str, Any] | None:
    """The search record of a ``PressureFitResult`` / ``LookaheadResult``; None for planners that keep none."""
    if hasattr(result, "diagnostics"):
        d = result.diagnostics()
        return {"planner": "pressurefit", "planning_s": d.planning_s, "selected": d.selected, "candidate_count": d.candidate_count,
                "valid": d.valid_candidate_count, "repaired": d.repaired_candidate_count, "early_exit": d.early_exit,
                "refined_moves": d.refined_moves, "spread": d.spread, "text": d.format(),
                "candidates": [{"name": c.name, "status": c.status, "makespan_us": c.makespan, "peak_fast_bytes": c.peak_fast,
                                "repairs": c.repairs, "wall_s": c.wall_s, "error": c.error} for c in d.candidates]}
    if hasattr(result, "candidates"):
        return {"planner": "lookahead", "selected": result.chosen.spec, "candidate_count": len(result.candidates),
                "candidates": [{"name": c.spec, "status": "failed" if c.makespan is None else "ok", "makespan_us": c.makespan,
                                "peak_fast_bytes": c.peak_fast, "emergencies": c.emergencies, "error": c.error}
                               for c in result.candidates]}
    return None
