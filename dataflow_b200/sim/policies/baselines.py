"""``all_resident``: the plan with no planning.  Everything that starts in backing memory is placed in fast memory up front
and nothing is evicted; it is the yardstick the budgets of the planner corpus are fractions of, and the plan to use when
the model simply fits.  The planners proper live beside this file: ``pressurefit`` and ``lookahead`` (what training uses),
``max_reduce``, ``min_grow``, ``roundtrip``, ``reactive`` (``belady_reactive``) and ``sliding_window``.
"""
from __future__ import annotations

from dataclasses import replace

from ..errors import SimulationCapacityError, SimulationError
from ..schema import Object, TaskChain, TransferTrigger
from ..simulator import Simulator
from .pressurefit import PlanningError, gather_facts


def _verified(chain: TaskChain, name: str) -> TaskChain:
    try:
        Simulator(chain).run()
    except (SimulationCapacityError, SimulationError) as e:
        raise PlanningError(f"{name}: {e}") from None
    return chain


def all_resident(chain: TaskChain, fast_memory_capacity: int | None = None) -> TaskChain:
    """Everything that starts in backing is placed in fast memory up front and nothing is evicted;
    objects are released (or written back, when they must end in backing) after their last use."""
    base = chain.bare()
    facts = gather_facts(base)
    initial = list(base.initial_memory)
    have_fast = {o.id for o in initial if o.location == "fast"}
    for f in facts.values():
        if f.birth == -1 and f.id not in have_fast and f.uses:
            initial.append(Object(f.id, f.size, "fast", f.type))
    tasks = [replace(t, releases_after=[], offload_after=[], prefetch_after=[]) for t in base.tasks]
    dirty = {f.id: (f.birth != -1 or not f.in_backing) for f in facts.values()}
    if tasks:
        for f in facts.values():
            # an initial fast object nothing reads: it leaves after the first task (written back when it must end in backing
            # memory and has no copy there)
            if f.birth == -1 and f.in_fast and not f.uses and f.final != "fast":
                if f.final == "backing" and not f.in_backing:
                    tasks[0].offload_after.append(TransferTrigger(f.id))
                else:
                    tasks[0].releases_after.append(f.id)
    for i, t in enumerate(base.tasks):
        for m in t.mutates_inputs:
            dirty[m] = True
        for x in t.outputs:
            # an output produced in backing memory that something reads later is fetched at once and stays
            if x.location == "backing" and len(facts[x.id].uses) > 1:
                tasks[i].prefetch_after.append(TransferTrigger(x.id))
                dirty[x.id] = False
        for o in dict.fromkeys(list(t.inputs) + [x.id for x in t.outputs if x.location == "fast"]):
            f = facts[o]
            if not f.uses or f.uses[-1] != i:
                continue
            if f.final == "fast":
                continue
            if f.final == "backing" and dirty.get(o, False):
                tasks[i].offload_after.append(TransferTrigger(o))
            else:
                tasks[i].releases_after.append(o)
    return _verified(replace(base, tasks=tasks, initial_memory=initial, fast_memory_capacity=fast_memory_capacity),
                     "all_resident")
