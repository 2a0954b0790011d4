"""What a traced step says about overlap, from the engine's own trace (intervals on the compute lane and the two copy
lanes): how much of each copy lane's busy time ran under compute, how much of the step had compute and a copy, compute
alone, a copy alone or nothing running, and the gaps of the compute lane split by cause (a late operand or dispatch).
The functions take ``runtime.trace`` intervals; ``trace_cell.py`` runs a cell and prints them."""
from __future__ import annotations

import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.join(ROOT, "tools", "bench"))


def _union(ivs) -> list[tuple[float, float]]:
    out: list[list[float]] = []
    for a, b in sorted((i.start_us, i.end_us) for i in ivs):
        if out and a <= out[-1][1]:
            out[-1][1] = max(out[-1][1], b)
        else:
            out.append([a, b])
    return [(a, b) for a, b in out]


def _length(u) -> float:
    return sum(b - a for a, b in u)


def _intersect(u, v) -> list[tuple[float, float]]:
    out, i, j = [], 0, 0
    while i < len(u) and j < len(v):
        a, b = max(u[i][0], v[j][0]), min(u[i][1], v[j][1])
        if a < b:
            out.append((a, b))
        if u[i][1] < v[j][1]:
            i += 1
        else:
            j += 1
    return out


def overlap_report(trace) -> dict:
    comp = _union(trace.by_track("compute"))
    lanes = {d: _union(trace.by_track(d)) for d in ("from_slow", "to_slow")}
    every = [i for i in trace.intervals]
    if not every:
        return {"span_us": 0.0}
    t0, t1 = min(i.start_us for i in every), max(i.end_us for i in every)
    span = t1 - t0
    copy = _union([i for d in ("from_slow", "to_slow") for i in trace.by_track(d)])
    both = _length(_intersect(comp, copy))
    out = {"span_us": span, "compute_busy_pct": 100.0 * _length(comp) / span, "copy_busy_pct": 100.0 * _length(copy) / span,
           "compute_and_copy_pct": 100.0 * both / span, "compute_only_pct": 100.0 * (_length(comp) - both) / span,
           "copy_only_pct": 100.0 * (_length(copy) - both) / span,
           "nothing_pct": 100.0 * (span - _length(comp) - _length(copy) + both) / span, "lanes": {}}
    for d, u in lanes.items():
        busy = _length(u)
        out["lanes"][d] = {"busy_us": busy, "busy_pct": 100.0 * busy / span, "transfers": len(trace.by_track(d)),
                           "hidden_under_compute_pct": 100.0 * _length(_intersect(u, comp)) / busy if busy else 100.0}
    out["both_directions_pct"] = 100.0 * _length(_intersect(lanes["from_slow"], lanes["to_slow"])) / span
    return out


def gap_report(program, trace, floor_us: float = 0.0) -> dict:
    from gap_census import census
    return census(program, trace, floor_us)
