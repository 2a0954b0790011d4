"""Where a plan's time went, from the simulator's own event log.

``build_stall_report(chain, log)`` answers: how long compute stalled in total, which tasks stalled and
whether each waited for an inbound transfer (and of which objects) or for fast-memory room, how busy
each copy lane was, and when a lane had work queued behind the transfer in flight (backlog).  Layered
planners (recompute selection) and the trace tools read this instead of re-deriving pressure from an
analytic model.  Role parity: reference ``src/dataflow_sim/engine/stall_report.py``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .schema import EventLog, TaskChain


@dataclass
class TaskStall:
    task_id: str
    index: int
    stall_us: float
    waited_inputs: tuple[str, ...]      # inputs not live when the task first blocked
    waited_capacity: bool               # fast memory could not admit its outputs / workspace
    blocking_object: str | None = None  # the input whose transfer finished last (it released the task)


@dataclass
class LaneUse:
    busy_us: float
    busy_fraction: float
    transfers: int
    backlog_us: float                   # time during which at least one more transfer was queued behind


@dataclass
class StallReport:
    makespan_us: float
    compute_us: float
    stall_us: float
    stalls: list[TaskStall] = field(default_factory=list)
    lanes: dict[str, LaneUse] = field(default_factory=dict)
    by_object_type: dict[str, float] = field(default_factory=dict)   # stall µs attributed to object roles

    @property
    def stall_fraction(self) -> float:
        return 0.0 if self.makespan_us <= 0 else self.stall_us / self.makespan_us

    def top(self, n: int = 10) -> list[TaskStall]:
        return sorted(self.stalls, key=lambda s: -s.stall_us)[:n]

    def format(self, n: int = 10) -> str:
        lines = [f"makespan {self.makespan_us / 1e3:.2f} ms, compute {self.compute_us / 1e3:.2f} ms, "
                 f"stalled {self.stall_us / 1e3:.2f} ms ({100 * self.stall_fraction:.1f} %)"]
        for name, l in self.lanes.items():
            lines.append(f"  {name}: busy {100 * l.busy_fraction:.1f} % over {l.transfers} transfers, "
                         f"backlog {l.backlog_us / 1e3:.2f} ms")
        for s in self.top(n):
            why = "capacity" if s.waited_capacity and not s.waited_inputs else f"inputs {list(s.waited_inputs)}"
            lines.append(f"  {s.task_id}: {s.stall_us / 1e3:.2f} ms waiting for {why}"
                         + (f" (last: {s.blocking_object})" if s.blocking_object else ""))
        return "\n".join(lines)


def build_stall_report(chain: TaskChain, log: EventLog) -> StallReport:
    index = {t.id: i for i, t in enumerate(chain.tasks)}
    types: dict[str, str] = {o.id: o.type for o in chain.initial_memory}
    for t in chain.tasks:
        for o in t.outputs:
            types[o.id] = o.type
    compute = [iv for iv in log.task_intervals if iv.track == "compute"]
    start_of = {iv.task_id: iv.start for iv in compute}
    compute_us = sum(iv.end - iv.start for iv in compute)
    inbound_end: dict[str, list[float]] = {}
    lanes: dict[str, LaneUse] = {}
    for lane in ("from_slow", "to_slow"):
        ivs = sorted((iv for iv in log.task_intervals if iv.track == lane), key=lambda iv: iv.start)
        busy = sum(iv.end - iv.start for iv in ivs)
        # FIFO lane, one in flight: the next transfer was waiting whenever it starts exactly at the previous end
        backlog = 0.0
        for a, b in zip(ivs, ivs[1:]):
            if abs(b.start - a.end) < 1e-9:
                backlog += a.end - a.start
        lanes[lane] = LaneUse(busy, busy / log.makespan if log.makespan else 0.0, len(ivs), backlog)
        if lane == "from_slow":
            for iv in ivs:
                obj = iv.task_id.split(":", 1)[1].split("#", 1)[0]
                inbound_end.setdefault(obj, []).append(iv.end)
    stalls: list[TaskStall] = []
    by_type: dict[str, float] = {}
    for tid, us in log.stalls.items():
        waited, short = log.stall_causes.get(tid, ((), False))
        blocker = None
        t0 = start_of.get(tid)
        if waited and t0 is not None:
            best = -1.0
            for o in waited:
                ends = [e for e in inbound_end.get(o, ()) if e <= t0 + 1e-9]
                if ends and max(ends) > best:
                    best, blocker = max(ends), o
        stalls.append(TaskStall(tid, index.get(tid, -1), us, tuple(waited), bool(short), blocker))
        key = types.get(blocker, "other") if blocker else ("capacity" if short else "other")
        by_type[key] = by_type.get(key, 0.0) + us
    stalls.sort(key=lambda s: s.index)
    return StallReport(log.makespan, compute_us, sum(log.stalls.values()), stalls, lanes, by_type)
