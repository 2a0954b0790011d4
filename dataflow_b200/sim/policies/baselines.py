"""Comparison planners.  Each takes ``(chain, fast_memory_capacity)`` and returns an annotated chain
that the simulator completes under the capacity (or raises ``PlanningError``).  They exist to
be compared against PressureFit / Lookahead in the planner panel and in tests; each is a small
construction on this repository's own planning machinery, not a rewrite of the reference's
(``src/dataflow_sim/policies/{sliding_window,belady_reactive,roundtrip_planner,max_reduce,
min_grow}.py`` — same names, same role: a hand pattern, a reactive Belady, a round-trip packer,
a residency-only reducer, and a search that uses the simulator as its oracle).
"""
from __future__ import annotations

from dataclasses import replace

from ..errors import SimulationCapacityError, SimulationError
from ..schema import Object, TaskChain, TransferTrigger
from ..simulator import Simulator
from .lookahead import LOOKAHEAD_SPECS, LookaheadSpec, _v_cost_aware, _v_farthest, plan_one
from .pressurefit import PREFETCH_RULES, RESIDENCY_SPECS, PlanningError, gather_facts, pressurefit


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
    for i, t in enumerate(base.tasks):
        for m in t.mutates_inputs:
            dirty[m] = True
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


def sliding_window(chain: TaskChain, fast_memory_capacity: int | None = None, window_size: int = 2) -> TaskChain:
    """The classic hand pattern, made generic over object roles: every long-lived object is evicted right
    after each use and fetched back ``window_size`` tasks before its next one (PressureFit's ``window``
    prefetch rule on a Belady residency, one candidate, no search)."""
    want = 1 if window_size <= 1 else 2 if window_size <= 3 else 4
    rule = next(r for r in PREFETCH_RULES if r.kind == "window" and int(r.param) == want)
    spec = next(s for s in RESIDENCY_SPECS if s.name == "belady")
    return pressurefit(chain, fast_memory_capacity, specs=[spec], rules=[rule], early_exit=False).chain


def belady_reactive(chain: TaskChain, fast_memory_capacity: int | None = None) -> TaskChain:
    """Reactive Belady inside the simulator: evict the resident needed farthest in the future only when the
    next task would not fit, fetch only what is about to be late."""
    spec = LookaheadSpec("reactive", _v_farthest, slack=1.0, evict_lead=0.0, early_room=0.0)
    try:
        planned, _, _ = plan_one(chain.bare(), fast_memory_capacity if fast_memory_capacity is not None
                                 else chain.fast_memory_capacity, spec, 0.0)
    except (SimulationCapacityError, SimulationError) as e:
        raise PlanningError(f"belady_reactive: {e}") from None
    return planned


def roundtrip_planner(chain: TaskChain, fast_memory_capacity: int | None = None) -> TaskChain:
    """Round trips for the objects with the widest idle gaps: bytes x distance residency with just-in-time
    reloads packed backwards on the ``from_slow`` lane."""
    specs = [s for s in RESIDENCY_SPECS if s.name == "bytes_x_distance"]
    rules = [r for r in PREFETCH_RULES if r.kind == "jit"]
    try:
        return pressurefit(chain, fast_memory_capacity, specs=specs, rules=rules).chain
    except PlanningError:
        return pressurefit(chain, fast_memory_capacity, specs=specs).chain


def max_reduce(chain: TaskChain, fast_memory_capacity: int | None = None) -> TaskChain:
    """Residency only, no timing: start from everything resident and remove the largest idle residents until
    every boundary fits; reloads one task ahead."""
    specs = [s for s in RESIDENCY_SPECS if s.name == "largest"]
    rules = [r for r in PREFETCH_RULES if r.name in ("window_1", "window_2")]
    return pressurefit(chain, fast_memory_capacity, specs=specs, rules=rules, early_exit=False).chain


def min_grow(chain: TaskChain, fast_memory_capacity: int | None = None, rounds: int = 3) -> TaskChain:
    """Search with the simulator as the oracle: coordinate descent over the Lookahead knobs (transfer slack,
    eviction lead, early-prefetch share, headroom), every point priced by a full simulated run."""
    cap = fast_memory_capacity if fast_memory_capacity is not None else chain.fast_memory_capacity
    base = chain.bare()

    def price(slack, lead, early, head):
        try:
            planned, log, _ = plan_one(base, cap, LookaheadSpec("search", _v_cost_aware, slack, lead, early), head)
            return log.makespan, planned
        except (SimulationCapacityError, SimulationError):
            return float("inf"), None

    point = [1.25, 2.0, 1.0, 0.02]
    grids = [(1.0, 1.25, 1.6, 2.5), (0.0, 1.0, 2.0, 4.0), (0.0, 0.5, 1.0), (0.0, 0.02, 0.05, 0.1)]
    best_ms, best = price(*point)
    for _ in range(rounds):
        moved = False
        for axis, grid in enumerate(grids):
            for v in grid:
                if v == point[axis]:
                    continue
                trial = list(point)
                trial[axis] = v
                ms, planned = price(*trial)
                if ms < best_ms - 1e-9:
                    best_ms, best, point, moved = ms, planned, trial, True
        if not moved:
            break
    if best is None:
        raise PlanningError(f"min_grow: no knob setting fits {cap} bytes")
    return best
