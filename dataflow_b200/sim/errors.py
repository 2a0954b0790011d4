"""Typed simulator failures.  The capacity error carries enough context for the
planner's physical-repair pass (reference ``src/dataflow_sim/engine/errors.py``)."""
from __future__ import annotations


class SimulationError(ValueError):
    """A plan that violates a directive-state rule (release of a non-live object …)."""


class SimulationCapacityError(SimulationError):
    def __init__(self, message: str, *, kind: str, task_id: str | None = None,
                 location: str = "fast", capacity_bytes: int | None = None,
                 actual_need_bytes: int | None = None, overage_bytes: int | None = None,
                 missing_object_ids: tuple[str, ...] = (), time: float | None = None,
                 resident: tuple[tuple[str, int], ...] = ()):
        super().__init__(message)
        self.kind = kind
        self.task_id = task_id
        self.location = location
        self.capacity_bytes = capacity_bytes
        self.actual_need_bytes = actual_need_bytes
        self.overage_bytes = overage_bytes
        self.missing_object_ids = tuple(missing_object_ids)
        self.time = time
        self.resident = tuple(resident)
