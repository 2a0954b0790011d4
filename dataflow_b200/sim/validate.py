"""Structural validation of TaskChains (reference ``src/dataflow_sim/core/validate.py:421-441``).

``validate_chain`` checks what the simulator would otherwise trip over half-way
through a run; ``validate_planning_input`` additionally demands a *bare* chain.
"""
from __future__ import annotations

from .schema import TaskChain


class ValidationError(ValueError):
    def __init__(self, problems):
        self.problems = list(problems)
        super().__init__("invalid chain:\n  - " + "\n  - ".join(self.problems))


def chain_problems(chain: TaskChain) -> list[str]:
    probs: list[str] = []
    sizes: dict[str, int] = {}
    seen: set[tuple[str, str]] = set()
    for o in chain.initial_memory:
        if o.location not in ("fast", "backing"):
            probs.append(f"object {o.id!r}: bad location {o.location!r}")
        if (o.id, o.location) in seen:
            probs.append(f"object {o.id!r} appears twice at {o.location!r}")
        seen.add((o.id, o.location))
        if o.size < 0:
            probs.append(f"object {o.id!r}: negative size")
        if o.id in sizes and sizes[o.id] != o.size:
            probs.append(f"object {o.id!r}: copies differ in size")
        sizes[o.id] = o.size
    ids: set[str] = set()
    need_from = need_to = False
    for t in chain.tasks:
        if t.id in ids:
            probs.append(f"duplicate task id {t.id!r}")
        ids.add(t.id)
        if t.runtime < 0:
            probs.append(f"task {t.id!r}: negative runtime")
        if t.workspace_bytes < 0:
            probs.append(f"task {t.id!r}: negative workspace")
        if len(set(t.inputs)) != len(t.inputs):
            probs.append(f"task {t.id!r}: repeated input")
        for i in t.inputs:
            if i not in sizes:
                probs.append(f"task {t.id!r}: input {i!r} unknown at this point")
        for m in t.mutates_inputs:
            if m not in t.inputs:
                probs.append(f"task {t.id!r}: mutated {m!r} is not an input")
        for o in t.outputs:
            if o.id in sizes:
                probs.append(f"task {t.id!r}: output {o.id!r} reuses an id")
            if o.size < 0:
                probs.append(f"task {t.id!r}: output {o.id!r} negative size")
            sizes[o.id] = o.size
        for r in t.releases_after:
            if r not in sizes:
                probs.append(f"task {t.id!r}: release of unknown {r!r}")
        for tr in t.offload_after:
            if tr.obj_id not in sizes:
                probs.append(f"task {t.id!r}: offload of unknown {tr.obj_id!r}")
            need_to |= tr.runtime is None
        for tr in t.prefetch_after:
            if tr.obj_id not in sizes:
                probs.append(f"task {t.id!r}: prefetch of unknown {tr.obj_id!r}")
            need_from |= tr.runtime is None
        dup = set(t.releases_after) & {x.obj_id for x in t.offload_after}
        if dup:
            probs.append(f"task {t.id!r}: {sorted(dup)} both released and offloaded")
    if need_from and not chain.bandwidth_from_slow:
        probs.append("prefetch triggers need bandwidth_from_slow")
    if need_to and not chain.bandwidth_to_slow:
        probs.append("offload triggers need bandwidth_to_slow")
    for o, loc in chain.final_locations.items():
        if o not in sizes:
            probs.append(f"final_locations: unknown object {o!r}")
        if loc not in ("fast", "backing"):
            probs.append(f"final_locations[{o!r}]: bad location")
    for cap in ("fast_memory_capacity", "backing_memory_capacity"):
        v = getattr(chain, cap)
        if v is not None and v < 0:
            probs.append(f"{cap} negative")
    return probs


def validate_chain(chain: TaskChain) -> TaskChain:
    probs = chain_problems(chain)
    if probs:
        raise ValidationError(probs)
    return chain


def validate_planning_input(chain: TaskChain) -> TaskChain:
    probs = chain_problems(chain)
    for t in chain.tasks:
        if t.releases_after or t.offload_after or t.prefetch_after:
            probs.append(f"task {t.id!r} already carries plan annotations")
            break
    if probs:
        raise ValidationError(probs)
    return chain
