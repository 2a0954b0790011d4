"""Executable ABI: what a task's implementation sees.

``Executable.launch(ctx)`` may only *enqueue* device work on ``ctx.stream``: no
host synchronisation, no device-to-host read-back, no data-dependent host
control flow, no vendor allocation.  Contract parity: reference
``src/dataflow/runtime/executable.py:30-77`` and ``docs/task-contract.md:55-93``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping, Protocol

from ..core import Program, TaskSpec


@dataclass(frozen=True)
class Buffer:
    """A raw extent handed to an executable (device or host address + byte size)."""
    ptr: int
    size: int
    location: str = "fast"
    object_id: str = ""


@dataclass
class TaskContext:
    task: TaskSpec
    stream: int                                  # raw stream handle (cudaStream_t) or 0 on host backends
    inputs: tuple[Buffer, ...]
    outputs: tuple[Buffer, ...]
    backend: Any
    run_args: Mapping[str, Any] = field(default_factory=dict)
    run_values: dict[str, Any] = field(default_factory=dict)
    groups: Mapping[str, Any] = field(default_factory=dict)
    workspace: Any = None

    @property
    def mutates(self) -> tuple[Buffer, ...]:
        names = set(self.task.mutates)
        return tuple(b for b in self.inputs if b.object_id in names)

    def input(self, object_id: str) -> Buffer:
        for b in self.inputs:
            if b.object_id == object_id:
                return b
        raise KeyError(object_id)


class Executable(Protocol):
    def launch(self, ctx: TaskContext) -> None: ...


class SyntheticExecutable:
    """Occupies the compute stream for the task's planned ``runtime_us``."""

    def launch(self, ctx: TaskContext) -> None:
        ctx.backend.busy(0, float(ctx.task.runtime_us))


Resolver = Callable[[TaskSpec], Executable]


def synthetic_resolver(task: TaskSpec) -> Executable:
    return SyntheticExecutable()
