"""Hardware-free workload programs ("dataflow-workload/v1") and their compiler to simulator chains.

A workload program names objects (bytes) and tasks; a task's cost is a list of sub-ops, each a hardware-free
quantity — tensor FLOPs of a dtype, bytes through device memory, bytes over the scale-up fabric, or a fixed time.
``resolve_cost`` prices a cost on a ``HardwareSpec``; ``preview_workload`` reports totals without choosing a plan;
``realize_workload`` returns the ``TaskChain`` the simulator and the planners consume.
Reference role: ``src/dataflow_sim/workloads/dataflow.py:45-255,382,582,628`` (pydantic ``DataflowProgram v1``,
``resolve_cost``, ``preview_dataflow_program``, ``realize_dataflow_program``).
"""
from __future__ import annotations

from typing import Literal

from pydantic import BaseModel, Field, model_validator

from ..schema import Object, OutputAlloc, Task, TaskChain
from .hardware import HardwareSpec

SCHEMA = "dataflow-workload/v1"


class SubOp(BaseModel):
    name: str = ""
    kind: Literal["matmul", "attention", "memory", "scale_up", "fixed"] = "matmul"
    flops: float = 0.0
    dtype: str = "bf16"
    bytes: float = 0.0
    runtime_us: float = 0.0
    efficiency: float | None = None          # overrides the hardware row's efficiency for this term


class WorkloadCost(BaseModel):
    ops: list[SubOp] = Field(default_factory=list)
    combine: Literal["sum", "max"] = "sum"


class WorkloadObject(BaseModel):
    id: str
    bytes: int
    location: Literal["fast", "backing"] = "backing"
    type: str = "other"


class WorkloadOutput(BaseModel):
    id: str
    bytes: int
    location: Literal["fast", "backing"] = "fast"
    type: str = "other"


class WorkloadTask(BaseModel):
    id: str
    inputs: list[str] = Field(default_factory=list)
    outputs: list[WorkloadOutput] = Field(default_factory=list)
    mutates: list[str] = Field(default_factory=list)
    cost: WorkloadCost = Field(default_factory=WorkloadCost)
    workspace_bytes: int = 0
    phase: str = ""                           # fwd | head | bwd | recompute | optimizer (for summaries)
    tokens: int = 0


class WorkloadProgram(BaseModel):
    schema_version: str = Field(default=SCHEMA, alias="schema")
    name: str = ""
    objects: list[WorkloadObject] = Field(default_factory=list)
    tasks: list[WorkloadTask] = Field(default_factory=list)
    final_locations: dict[str, Literal["fast", "backing"]] = Field(default_factory=dict)
    metadata: dict = Field(default_factory=dict)

    model_config = {"populate_by_name": True}

    @model_validator(mode="after")
    def _check(self):
        if self.schema_version != SCHEMA:
            raise ValueError(f"unsupported workload schema {self.schema_version!r} (want {SCHEMA!r})")
        known = {o.id for o in self.objects}
        if len(known) != len(self.objects):
            raise ValueError("duplicate object id in `objects`")
        seen_tasks = set()
        for t in self.tasks:
            if t.id in seen_tasks:
                raise ValueError(f"duplicate task id {t.id!r}")
            seen_tasks.add(t.id)
            for i in t.inputs:
                if i not in known:
                    raise ValueError(f"task {t.id!r} reads {i!r} before anything produced it")
            for m in t.mutates:
                if m not in t.inputs:
                    raise ValueError(f"task {t.id!r} mutates {m!r} which is not among its inputs")
            for o in t.outputs:
                if o.id in known:
                    raise ValueError(f"task {t.id!r} re-creates object {o.id!r}")
                known.add(o.id)
        for oid in self.final_locations:
            if oid not in known:
                raise ValueError(f"final location names unknown object {oid!r}")
        return self


def resolve_subop(op: SubOp, hw: HardwareSpec) -> float:
    """Microseconds of one sub-op on ``hw`` (launch cost included)."""
    if op.kind == "fixed":
        return float(op.runtime_us)
    if op.kind in ("matmul", "attention"):
        eff = op.efficiency if op.efficiency is not None else (hw.matmul_efficiency if op.kind == "matmul" else hw.attention_efficiency)
        t = op.flops / (hw.tflops(op.dtype) * 1e12 * max(eff, 1e-6)) * 1e6
        # a tensor op cannot beat streaming its operands once
        if op.bytes:
            t = max(t, op.bytes / (hw.hbm_gbs * 1e9 * hw.memory_efficiency) * 1e6)
        return t + hw.launch_us
    if op.kind == "memory":
        eff = op.efficiency if op.efficiency is not None else hw.memory_efficiency
        return op.bytes / (hw.hbm_gbs * 1e9 * max(eff, 1e-6)) * 1e6 + hw.launch_us
    if op.kind == "scale_up":
        if hw.scale_up_bw_gbs <= 0:
            raise ValueError(f"hardware {hw.name!r} has no scale-up fabric but the workload has a collective ({op.name!r})")
        return op.bytes / (hw.scale_up_bw_gbs * 1e9 * (op.efficiency or 0.8)) * 1e6 + hw.launch_us
    raise ValueError(f"unknown sub-op kind {op.kind!r}")


def resolve_cost(cost: WorkloadCost, hw: HardwareSpec) -> float:
    times = [resolve_subop(op, hw) for op in cost.ops]
    if not times:
        return 0.0
    return max(times) if cost.combine == "max" else sum(times)


def cost_breakdown(cost: WorkloadCost, hw: HardwareSpec) -> list[dict]:
    return [{"name": op.name, "kind": op.kind, "us": resolve_subop(op, hw), "flops": op.flops, "bytes": op.bytes} for op in cost.ops]


def preview_workload(prog: WorkloadProgram, hw: HardwareSpec) -> dict:
    """Plan-free totals: compute-only lower bound, FLOPs, bytes of state and activations, tokens."""
    total_us, flops, by_phase = 0.0, 0.0, {}
    for t in prog.tasks:
        us = resolve_cost(t.cost, hw)
        total_us += us
        f = sum(op.flops for op in t.cost.ops)
        flops += f
        ph = by_phase.setdefault(t.phase or "other", {"us": 0.0, "flops": 0.0, "tasks": 0})
        ph["us"] += us
        ph["flops"] += f
        ph["tasks"] += 1
    initial = sum(o.bytes for o in prog.objects)
    produced = sum(o.bytes for t in prog.tasks for o in t.outputs)
    return {"name": prog.name, "tasks": len(prog.tasks), "objects": len(prog.objects) + sum(len(t.outputs) for t in prog.tasks),
            "compute_only_us": total_us, "total_flops": flops, "initial_bytes": initial, "produced_bytes": produced,
            "largest_workspace_bytes": max((t.workspace_bytes for t in prog.tasks), default=0),
            "tokens": int(prog.metadata.get("tokens_per_step", 0)), "by_phase": by_phase,
            "hardware": hw.name}


def realize_workload(prog: WorkloadProgram, hw: HardwareSpec, fast_memory_bytes: int | None = None) -> TaskChain:
    """The hardware-resolved chain (bare: no transfer directives) for the simulator and the planners."""
    tasks = [Task(id=t.id, inputs=list(t.inputs),
                  outputs=[OutputAlloc(o.id, int(o.bytes), o.location, o.type) for o in t.outputs],
                  runtime=resolve_cost(t.cost, hw), workspace_bytes=int(t.workspace_bytes), mutates_inputs=list(t.mutates))
             for t in prog.tasks]
    cap = fast_memory_bytes if fast_memory_bytes is not None else int(hw.fast_memory_gib * (1 << 30))
    return TaskChain(initial_memory=[Object(o.id, int(o.bytes), o.location, o.type) for o in prog.objects], tasks=tasks,
                     final_locations=dict(prog.final_locations), fast_memory_capacity=cap,
                     bandwidth_from_slow=int(hw.from_slow_gbs * 1e3), bandwidth_to_slow=int(hw.to_slow_gbs * 1e3))
