"""Forward reference tape: for every object the remaining tasks touch (read as an input or allocate as an
output), the time of the first touch — the next-use oracle Belady-style planners consult.
Role parity: reference ``src/dataflow_sim/core/reference_stream.py``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Mapping

from .schema import Task


@dataclass(frozen=True)
class Reference:
    obj_id: str
    ref_t: float
    ref_task: str


def compute_reference_stream(remaining_tasks: Iterable[Task], task_start_times: Mapping[str, float]) -> list[Reference]:
    first: dict[str, Reference] = {}
    for task in remaining_tasks:
        t = task_start_times[task.id]
        for oid in list(task.inputs) + [o.id for o in task.outputs]:
            if oid not in first:
                first[oid] = Reference(oid, t, task.id)
    return sorted(first.values(), key=lambda r: (r.ref_t, r.obj_id))


def next_ref_time(obj_id: str, remaining_tasks: Iterable[Task], task_start_times: Mapping[str, float]) -> float | None:
    for task in remaining_tasks:
        if obj_id in task.inputs or any(o.id == obj_id for o in task.outputs):
            return task_start_times[task.id]
    return None


def stall_free_starts(tasks: Iterable[Task], t0: float = 0.0) -> dict[str, float]:
    out, t = {}, t0
    for task in tasks:
        out[task.id] = t
        t += task.runtime
    return out
