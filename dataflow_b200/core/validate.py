"""Static validation of a Program.  All problems are collected, then raised once.

Rule catalogue (reference ``src/dataflow/core/validate.py:25-140``): unique ids
per location, inputs exist before use, ``mutates ⊆ inputs``, fresh output ids,
legal directive targets, bandwidth present when a directive needs it, rewrite
references resolve, dense TensorMeta agrees with ``size_bytes``.
"""
from __future__ import annotations

from .program import Program
from .types import DTYPE_BITS, LOCATIONS


class ValidationError(ValueError):
    def __init__(self, problems: list[str]):
        self.problems = list(problems)
        head = f"{len(problems)} problem(s) in program"
        super().__init__(head + ":\n  - " + "\n  - ".join(problems))


def _check_tensor(where: str, spec, problems: list[str]) -> None:
    t = spec.tensor
    if t is None or t.dtype is None or t.shape is None:
        return
    if t.dtype not in DTYPE_BITS:
        problems.append(f"{where}: unknown dtype {t.dtype!r}")
        return
    if any(int(s) < 0 for s in t.shape):
        problems.append(f"{where}: negative dimension in shape {t.shape}")
        return
    if t.strides is not None and len(t.strides) != len(t.shape):
        problems.append(f"{where}: strides rank {len(t.strides)} != shape rank {len(t.shape)}")
        return
    if t.is_dense() and t.nbytes() > spec.size_bytes:
        problems.append(f"{where}: dense tensor needs {t.nbytes()} bytes but object holds {spec.size_bytes}")


def collect_problems(p: Program) -> list[str]:
    problems: list[str] = []
    known: dict[str, int] = {}            # object id -> size
    seen_loc: set[tuple[str, str]] = set()
    for o in p.initial_objects:
        if o.location not in LOCATIONS:
            problems.append(f"initial object {o.id!r}: bad location {o.location!r}")
        if (o.id, o.location) in seen_loc:
            problems.append(f"initial object {o.id!r} listed twice at {o.location!r}")
        seen_loc.add((o.id, o.location))
        if o.id in known and known[o.id] != o.size_bytes:
            problems.append(f"initial object {o.id!r}: fast/backing copies differ in size")
        if o.size_bytes < 0:
            problems.append(f"initial object {o.id!r}: negative size")
        known[o.id] = o.size_bytes
        _check_tensor(f"initial object {o.id!r}", o, problems)

    task_ids: set[str] = set()
    needs_bw_from = needs_bw_to = False
    any_host = any_dev = False
    initial_ids = {o.id for o in p.initial_objects}
    for t in p.tasks:
        if t.id in task_ids:
            problems.append(f"duplicate task id {t.id!r}")
        task_ids.add(t.id)
        any_host |= t.host
        any_dev |= not t.host
        if t.runtime_us < 0:
            problems.append(f"task {t.id!r}: negative runtime_us")
        if t.workspace_bytes < 0:
            problems.append(f"task {t.id!r}: negative workspace_bytes")
        if len(set(t.inputs)) != len(t.inputs):
            problems.append(f"task {t.id!r}: repeated input id")
        for i in t.inputs:
            if i not in known:
                problems.append(f"task {t.id!r}: input {i!r} does not exist yet")
        for m in t.mutates:
            if m not in t.inputs:
                problems.append(f"task {t.id!r}: mutates {m!r} which is not an input")
        if t.host:
            if t.outputs:
                problems.append(f"host task {t.id!r} may not declare outputs")
            for i in t.inputs:
                if i not in initial_ids:
                    problems.append(f"host task {t.id!r}: {i!r} is not an initial object")
        for out in t.outputs:
            if out.id in known:
                problems.append(f"task {t.id!r}: output id {out.id!r} is not fresh")
            if out.location not in LOCATIONS:
                problems.append(f"task {t.id!r}: output {out.id!r} bad location {out.location!r}")
            if out.size_bytes < 0:
                problems.append(f"task {t.id!r}: output {out.id!r} negative size")
            known[out.id] = out.size_bytes
            _check_tensor(f"task {t.id!r} output {out.id!r}", out, problems)
        for r in t.releases_after:
            if r not in known:
                problems.append(f"task {t.id!r}: releases unknown object {r!r}")
        for d in t.offload_after:
            if d.object_id not in known:
                problems.append(f"task {t.id!r}: offloads unknown object {d.object_id!r}")
            needs_bw_to |= d.runtime_us is None
        for d in t.prefetch_after:
            if d.object_id not in known:
                problems.append(f"task {t.id!r}: prefetches unknown object {d.object_id!r}")
            needs_bw_from |= d.runtime_us is None
        if len(set(t.releases_after)) != len(t.releases_after):
            problems.append(f"task {t.id!r}: repeated release")
        both = set(t.releases_after) & {d.object_id for d in t.offload_after}
        for b in sorted(both):
            problems.append(f"task {t.id!r}: {b!r} is both released and offloaded")
    if any_host and any_dev:
        problems.append("program mixes host and device tasks")
    if needs_bw_from and not p.bandwidth_from_slow:
        problems.append("prefetch directives present but bandwidth_from_slow is unset")
    if needs_bw_to and not p.bandwidth_to_slow:
        problems.append("offload directives present but bandwidth_to_slow is unset")
    for obj, loc in p.final_locations.items():
        if obj not in known:
            problems.append(f"final_locations names unknown object {obj!r}")
        if loc not in LOCATIONS:
            problems.append(f"final_locations[{obj!r}]: bad location {loc!r}")
    for cap_name in ("fast_memory_capacity", "backing_memory_capacity"):
        cap = getattr(p, cap_name)
        if cap is not None and cap < 0:
            problems.append(f"{cap_name} is negative")
    for rw in p.recompute_rewrites:
        if rw.object_id not in known:
            problems.append(f"recompute rewrite names unknown object {rw.object_id!r}")
        if rw.f_task_id not in task_ids:
            problems.append(f"recompute rewrite for {rw.object_id!r}: unknown f_task {rw.f_task_id!r}")
        if not rw.options:
            problems.append(f"recompute rewrite for {rw.object_id!r} has no options")
        levels = [o.level for o in rw.options]
        if len(set(levels)) != len(levels):
            problems.append(f"recompute rewrite for {rw.object_id!r}: repeated level")
    return problems


def validate_program(p: Program) -> Program:
    problems = collect_problems(p)
    if problems:
        raise ValidationError(problems)
    return p
