"""Run traces and the engine-vs-simulator parity oracle.

Every run records one interval per task and per transfer (always on: two
events each).  ``compare_to_sim_eventlog`` is the check that the executor on the
virtual-time backend reproduces the planner's simulator exactly.  Parity:
reference ``src/dataflow/runtime/trace.py:14-141``.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any


@dataclass(frozen=True)
class Interval:
    name: str
    track: str          # compute | from_slow | to_slow
    start_us: float
    end_us: float


@dataclass(frozen=True)
class TraceEvent:
    kind: str
    what: str
    fast_bytes: int


@dataclass
class RunTrace:
    intervals: list[Interval] = field(default_factory=list)
    events: list[TraceEvent] = field(default_factory=list)
    peak_fast_bytes: int = 0
    peak_backing_bytes: int = 0

    def by_track(self, track: str) -> list[Interval]:
        return [i for i in self.intervals if i.track == track]

    def busy_us(self, track: str) -> float:
        return sum(i.end_us - i.start_us for i in self.by_track(track))


def trace_to_dict(trace: RunTrace) -> dict[str, Any]:
    return {"intervals": [asdict(i) for i in trace.intervals],
            "events": [asdict(e) for e in trace.events],
            "peak_fast_bytes": trace.peak_fast_bytes, "peak_backing_bytes": trace.peak_backing_bytes}


def trace_from_dict(d: dict[str, Any]) -> RunTrace:
    return RunTrace([Interval(**i) for i in d.get("intervals", [])],
                    [TraceEvent(**e) for e in d.get("events", [])],
                    d.get("peak_fast_bytes", 0), d.get("peak_backing_bytes", 0))


def compare_to_sim_eventlog(trace: RunTrace, log, *, tol_us: float = 1e-6) -> list[str]:
    """Differences between an engine trace and a simulator EventLog (empty list = parity)."""
    diffs: list[str] = []
    sim = {iv.task_id: iv for iv in log.task_intervals}
    eng = {iv.name: iv for iv in trace.intervals}
    for name in sim.keys() - eng.keys():
        diffs.append(f"simulator has {name!r}, engine does not")
    for name in eng.keys() - sim.keys():
        diffs.append(f"engine has {name!r}, simulator does not")
    for name in sim.keys() & eng.keys():
        s, e = sim[name], eng[name]
        if abs(s.start - e.start_us) > tol_us or abs(s.end - e.end_us) > tol_us:
            diffs.append(f"{name!r}: simulator [{s.start}, {s.end}] vs engine [{e.start_us}, {e.end_us}]")
        if s.track != e.track:
            diffs.append(f"{name!r}: track {s.track!r} vs {e.track!r}")
    if trace.peak_fast_bytes != log.peak_fast_memory_bytes:
        diffs.append(f"peak fast bytes: simulator {log.peak_fast_memory_bytes} vs engine {trace.peak_fast_bytes}")
    return sorted(diffs)
