"""Bridges between the core Program and the simulator's TaskChain.

The simulator package is imported lazily so ``dataflow_b200.core`` stays
stdlib-only at import time (reference ``src/dataflow/core/convert.py:53-344``).
"""
from __future__ import annotations

from dataclasses import replace
from typing import Any

from .program import (ObjectSpec, OutputSpec, Program, TaskSpec, TransferDirective)

_ROLE_TO_TYPE = {"parameter": "weight", "gradient": "gradient", "optimizer_state": "optimizer",
                 "activation": "activation"}
_TYPE_TO_ROLE = {v: k for k, v in _ROLE_TO_TYPE.items()}


def to_sim_chain(program: Program, *, with_directives: bool = True):
    """Program → TaskChain (sizes, runtimes, capacities and, if present, the plan)."""
    from ..sim.schema import Object, OutputAlloc, Task, TaskChain, TransferTrigger
    tasks = []
    for t in program.tasks:
        tasks.append(Task(
            id=t.id, inputs=list(t.inputs),
            outputs=[OutputAlloc(o.id, int(o.size_bytes), o.location, _ROLE_TO_TYPE.get(o.role, "other"))
                     for o in t.outputs],
            runtime=float(t.runtime_us), workspace_bytes=int(t.workspace_bytes),
            releases_after=list(t.releases_after) if with_directives else [],
            offload_after=[TransferTrigger(d.object_id, d.runtime_us) for d in t.offload_after] if with_directives else [],
            prefetch_after=[TransferTrigger(d.object_id, d.runtime_us) for d in t.prefetch_after] if with_directives else [],
            mutates_inputs=list(t.mutates)))
    return TaskChain(
        initial_memory=[Object(o.id, int(o.size_bytes), o.location, _ROLE_TO_TYPE.get(o.role, "other"))
                        for o in program.initial_objects],
        tasks=tasks, final_locations=dict(program.final_locations),
        fast_memory_capacity=program.fast_memory_capacity,
        backing_memory_capacity=program.backing_memory_capacity,
        bandwidth_from_slow=program.bandwidth_from_slow, bandwidth_to_slow=program.bandwidth_to_slow)


def apply_chain_annotations(program: Program, chain) -> Program:
    """Copy a planned chain's directives (and initial placements, capacities) onto the Program.

    Tasks are matched by id, so planner-inserted or dropped tasks are an error here:
    recompute variants must be re-lowered before planning.
    """
    by_id = {t.id: t for t in chain.tasks}
    if set(by_id) != {t.id for t in program.tasks}:
        missing = {t.id for t in program.tasks} ^ set(by_id)
        raise ValueError(f"chain and program disagree on task ids: {sorted(missing)[:6]}")
    new_tasks = []
    for t in program.tasks:
        c = by_id[t.id]
        new_tasks.append(replace(
            t, runtime_us=float(c.runtime),
            releases_after=tuple(c.releases_after),
            offload_after=tuple(TransferDirective(x.obj_id, x.runtime) for x in c.offload_after),
            prefetch_after=tuple(TransferDirective(x.obj_id, x.runtime) for x in c.prefetch_after)))
    spec = {}
    for o in program.initial_objects:
        spec.setdefault(o.id, o)
    initial = tuple(replace(spec[o.id], location=o.location, size_bytes=int(o.size)) for o in chain.initial_memory)
    return replace(program, tasks=tuple(new_tasks), initial_objects=initial,
                   fast_memory_capacity=chain.fast_memory_capacity,
                   backing_memory_capacity=chain.backing_memory_capacity,
                   bandwidth_from_slow=chain.bandwidth_from_slow,
                   bandwidth_to_slow=chain.bandwidth_to_slow,
                   final_locations=dict(chain.final_locations))


def from_sim_chain(chain, name: str = "chain") -> Program:
    """TaskChain → Program (synthetic executables; used by engine gates and tools)."""
    tasks = tuple(TaskSpec(
        id=t.id, inputs=tuple(t.inputs),
        outputs=tuple(OutputSpec(o.id, int(o.size), o.location, _TYPE_TO_ROLE.get(o.type, "other")) for o in t.outputs),
        mutates=tuple(t.mutates_inputs), runtime_us=float(t.runtime), workspace_bytes=int(t.workspace_bytes),
        releases_after=tuple(t.releases_after),
        offload_after=tuple(TransferDirective(x.obj_id, x.runtime) for x in t.offload_after),
        prefetch_after=tuple(TransferDirective(x.obj_id, x.runtime) for x in t.prefetch_after)) for t in chain.tasks)
    return Program(
        name=name,
        initial_objects=tuple(ObjectSpec(o.id, int(o.size), o.location, _TYPE_TO_ROLE.get(o.type, "other"))
                              for o in chain.initial_memory),
        tasks=tasks, final_locations=dict(chain.final_locations),
        fast_memory_capacity=chain.fast_memory_capacity, backing_memory_capacity=chain.backing_memory_capacity,
        bandwidth_from_slow=chain.bandwidth_from_slow, bandwidth_to_slow=chain.bandwidth_to_slow)


def to_webapp_program(program: Program) -> dict[str, Any]:
    """Hardware-free ``dataflow/v1`` upload document for the simulator web app.

    A task's ``metadata["cost_subops"]`` (list of ``{name, flops, memory_bytes, efficiency}``
    or ``{name, runtime_us}``) becomes a ``sum`` cost; otherwise the task is a fixed cost.
    """
    blocks: dict[str, dict[str, Any]] = {}
    tasks = []
    for t in program.tasks:
        subops = t.metadata.get("cost_subops") if t.metadata else None
        key = t.compute_block_key or t.id
        if subops:
            terms = []
            for s in subops:
                if "runtime_us" in s and "flops" not in s:
                    terms.append({"kind": "fixed", "name": s.get("name", ""), "runtime_us": s["runtime_us"]})
                else:
                    terms.append({"kind": "roofline", "name": s.get("name", ""), "flops": s.get("flops", 0),
                                  "memory_bytes": s.get("memory_bytes", 0),
                                  "dtype": s.get("dtype", "bf16"), "efficiency": s.get("efficiency", "matmul")})
            cost = {"kind": "sum", "terms": terms}
        else:
            cost = {"kind": "fixed", "runtime_us": t.runtime_us}
        sig = key if subops else f"{key}@{t.runtime_us}"
        blocks.setdefault(sig, {"key": sig, "name": key, "category": t.group, "cost": cost})
        tasks.append({"id": t.id, "label": t.label or t.id, "group": t.group, "compute_block_key": sig,
                      "inputs": list(t.inputs), "mutates": list(t.mutates),
                      "workspace_bytes": t.workspace_bytes,
                      "outputs": [{"id": o.id, "size_bytes": o.size_bytes, "location": o.location, "role": o.role}
                                  for o in t.outputs]})
    doc = {
        "schema_version": "dataflow/v1", "name": program.name,
        "objects": [{"id": o.id, "size_bytes": o.size_bytes, "initial_location": o.location, "role": o.role}
                    for o in program.initial_objects],
        "compute_blocks": list(blocks.values()), "tasks": tasks,
        "final_locations": dict(program.final_locations),
    }
    m = program.metadata or {}
    if "tokens_per_step" in m:
        doc["metrics"] = {"primary_unit": "tokens", "primary_count": m["tokens_per_step"]}
    return doc
