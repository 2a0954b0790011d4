"""Simulator-side chain schema (hardware-resolved, planner-facing).

Same vocabulary as the reference's ``src/dataflow_sim/core/schema.py:22-146``
(``Object``, ``OutputAlloc``, ``TransferTrigger``, ``Task``, ``TaskChain``,
``EventLog``) so converted chains and saved plans are interchangeable.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field, replace
from pathlib import Path
from typing import Any, Literal

Time = float
Location = Literal["backing", "fast"]
TransferDirection = Literal["from_slow", "to_slow"]
MEMORY_STATES = ("live", "reserved", "pending_inbound", "inbound", "pending_outbound", "outbound")


@dataclass(frozen=True)
class Object:
    id: str
    size: int
    location: Location = "fast"
    type: str = "other"


@dataclass(frozen=True)
class OutputAlloc:
    id: str
    size: int
    location: Location = "fast"
    type: str = "other"


@dataclass(frozen=True)
class TransferTrigger:
    obj_id: str
    runtime: Time | None = None


@dataclass(frozen=True)
class Task:
    id: str
    inputs: list[str]
    outputs: list[OutputAlloc]
    runtime: Time
    workspace_bytes: int = 0
    releases_after: list[str] = field(default_factory=list)
    offload_after: list[TransferTrigger] = field(default_factory=list)
    prefetch_after: list[TransferTrigger] = field(default_factory=list)
    mutates_inputs: list[str] = field(default_factory=list)

    def bare(self) -> "Task":
        return replace(self, releases_after=[], offload_after=[], prefetch_after=[])


@dataclass(frozen=True)
class TaskChain:
    initial_memory: list[Object]
    tasks: list[Task]
    final_locations: dict[str, Location] = field(default_factory=dict)
    fast_memory_capacity: int | None = None
    backing_memory_capacity: int | None = None
    bandwidth_from_slow: int | None = None
    bandwidth_to_slow: int | None = None

    def sizes(self) -> dict[str, int]:
        s = {o.id: o.size for o in self.initial_memory}
        for t in self.tasks:
            for o in t.outputs:
                s[o.id] = o.size
        return s

    def bare(self) -> "TaskChain":
        return replace(self, tasks=[t.bare() for t in self.tasks])

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "TaskChain":
        def trig(x):
            if isinstance(x, str):
                return TransferTrigger(x)
            return TransferTrigger(x.get("obj_id", x.get("id")), x.get("runtime"))
        return TaskChain(
            initial_memory=[Object(o["id"], int(o["size"]), o.get("location", "fast"), o.get("type", "other"))
                            for o in d.get("initial_memory", [])],
            tasks=[Task(id=t["id"], inputs=list(t.get("inputs", [])),
                        outputs=[OutputAlloc(o["id"], int(o["size"]), o.get("location", "fast"), o.get("type", "other"))
                                 for o in t.get("outputs", [])],
                        runtime=float(t["runtime"]), workspace_bytes=int(t.get("workspace_bytes", 0)),
                        releases_after=list(t.get("releases_after", [])),
                        offload_after=[trig(x) for x in t.get("offload_after", [])],
                        prefetch_after=[trig(x) for x in t.get("prefetch_after", [])],
                        mutates_inputs=list(t.get("mutates_inputs", [])))
                   for t in d.get("tasks", [])],
            final_locations=dict(d.get("final_locations", {})),
            fast_memory_capacity=d.get("fast_memory_capacity"),
            backing_memory_capacity=d.get("backing_memory_capacity"),
            bandwidth_from_slow=d.get("bandwidth_from_slow"),
            bandwidth_to_slow=d.get("bandwidth_to_slow"))

    def save(self, path) -> None:
        Path(path).write_text(json.dumps(self.to_dict(), indent=1))

    @staticmethod
    def load(path) -> "TaskChain":
        return TaskChain.from_dict(json.loads(Path(path).read_text()))


@dataclass(frozen=True)
class TaskInterval:
    task_id: str
    start: Time
    end: Time
    track: str = "compute"        # compute | from_slow | to_slow


@dataclass(frozen=True)
class Event:
    t: Time
    kind: str
    task_id: str | None = None
    transfer_obj: str | None = None
    transfer_direction: str | None = None
    object_ids: tuple[str, ...] = ()
    fast_bytes: int = 0
    backing_bytes: int = 0


@dataclass(frozen=True)
class MemoryTracePoint:
    t: Time
    fast_bytes: int
    workspace_bytes: int = 0


@dataclass
class EventLog:
    task_intervals: list[TaskInterval]
    events: list[Event]
    peak_fast_memory_bytes: int
    peak_backing_memory_bytes: int = 0
    memory_trace: list[MemoryTracePoint] = field(default_factory=list)
    stalls: dict[str, float] = field(default_factory=dict)     # task id -> µs waited after compute was free
    # task id -> (input objects that were not live when the task first blocked, short of fast memory?)
    stall_causes: dict[str, tuple[tuple[str, ...], bool]] = field(default_factory=dict)

    @property
    def makespan(self) -> Time:
        return max((iv.end for iv in self.task_intervals), default=0.0)

    def compute_intervals(self) -> list[TaskInterval]:
        return [iv for iv in self.task_intervals if iv.track == "compute"]

    def transfer_intervals(self, direction: str | None = None) -> list[TaskInterval]:
        return [iv for iv in self.task_intervals
                if iv.track != "compute" and (direction is None or iv.track == direction)]
