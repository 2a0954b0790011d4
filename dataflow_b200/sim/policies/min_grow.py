"""min_grow: start from the least residency that can run and grow it, with the simulator deciding what counts.

The seed is ``SpanPlan.fill_min(0)``: every object is in fast memory only during the tasks that touch it, so every idle gap
is a round trip through backing memory and every fetch is fired at the last moment.  If even that does not fit, nothing does, and that is the only infeasibility this
planner reports on its own.  Growth then removes round trips:

    static fill      every idle gap of every object is an offer "stay resident across the gap": its value is the lane time
                     it saves (a fetch, and an offload when the fast copy is the only current one).  Every fetch is an
                     offer "open the span early enough to arrive in time": its value is the stall it saves.  The price of
                     an offer is the bytes x time it occupies.  Offers are taken in order of value per price while the
                     level stays under the working capacity (a knapsack filled greedily; a lead may be taken in part).
    beam             the static fill has knobs the accounting cannot set by itself: how much of the capacity to leave for
                     bytes in flight (headroom), how much earlier than its own transfer time a fetch is fired (slack), and
                     whether price counts tasks or time.  A grid of knob settings is priced by full simulated runs and the
                     best ``beam`` plans survive.
    stall repair     for each survivor, the run's stall report names the tasks that waited for operands; the spans of those
                     operands are opened earlier (twice the lead, as far as the level allows) or merged with the span before,
                     and the plan is kept when the simulated makespan improves.  A few rounds, survivors re-ranked each time.

Reference role: ``src/dataflow_sim/policies/min_grow.py`` (plan search priced by simulator replay, beam over candidates).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from ..errors import SimulationCapacityError, SimulationError
from ..schema import TaskChain
from ..simulator import Simulator
from .pressurefit import PlanningError
from .spans import SpanPlan, check_input


@dataclass(frozen=True)
class GrowKnobs:
    headroom: float = 0.02
    slack: float = 1.25
    price: str = "time"          # what an offer pays per byte held: "time" (microseconds of the gap) or "tasks"


def offers(plan: SpanPlan, knobs: GrowKnobs) -> list[tuple[float, str, str, int, int]]:
    """(value per price, kind, object, first task, last task), best first.  Kind ``gap``: stay resident across an idle gap
    (saves the round trip); kind ``lead``: open a span early enough for its fetch to arrive in time (saves the stall)."""
    out = []
    by_time = knobs.price == "time"
    for o, spans in plan.spans.items():
        size = plan.facts[o].size
        if size <= 0:
            continue
        for (a0, b0), (a1, b1) in zip(spans, spans[1:]):
            lo, hi = b0 + 1, a1 - 1
            saved = plan.tau_in(o) + (0.0 if plan.clean_until(o, b0) else plan.tau_out(o))
            held = (plan.cum[hi + 1] - plan.cum[lo]) if by_time else float(hi - lo + 1)
            out.append((saved / max(size * held, 1e-9), "gap", o, lo, hi))
        for k, (a, b) in enumerate(spans):
            if k == 0 and plan.pinned_start[o]:
                continue
            floor = spans[k - 1][1] + 1 if k > 0 else plan.first_legal[o]
            lo = max(plan.lead_start(o, a, knobs.slack), floor)
            if lo < a:
                held = (plan.cum[a] - plan.cum[lo]) if by_time else float(a - lo)
                out.append((plan.tau_in(o) / max(size * held, 1e-9), "lead", o, lo, a - 1))
    out.sort(key=lambda x: -x[0])
    return out


def grow_static(chain: TaskChain, cap: int | None, knobs: GrowKnobs) -> SpanPlan:
    plan = SpanPlan(chain).fill_min(0.0)                         # spans of exactly the touching tasks: nothing less can run
    if cap is not None and float(plan.level.max(initial=0.0)) > cap:
        i = int(np.argmax(plan.level))
        raise PlanningError(f"min_grow: even the least residency needs {plan.level[i]:.0f} bytes during task "
                            f"{chain.tasks[i].id!r}, capacity {cap}")
    work = None if cap is None else cap * (1.0 - knobs.headroom)
    for _, kind, o, lo, hi in offers(plan, knobs):
        size = plan.facts[o].size
        if work is None or float(plan.level[lo:hi + 1].max()) + size <= work:
            plan.add(o, lo, hi)
        elif kind == "lead":                                     # as much of the lead as fits, from the use backwards
            a = hi + 1
            while a > lo and plan.level[a - 1] + size <= work:
                a -= 1
            if a <= hi:
                plan.add(o, a, hi)
    _preplace(plan, work)
    return plan


def _preplace(plan: SpanPlan, work: float | None) -> None:
    """Initial backing objects whose first span can be stretched back to task 0 start in fast memory: no fetch at all."""
    first = sorted(((plan.spans[o][0][0], o) for o, f in plan.facts.items()
                    if f.birth < 0 and not f.in_fast and plan.spans[o] and plan.spans[o][0][0] > 0))
    for a, o in first:
        if work is None or float(plan.level[0:a].max()) + plan.facts[o].size <= work:
            plan.add(o, 0, a - 1)


def _simulate(plan: SpanPlan, cap: int | None):
    try:
        planned = plan.emit(cap)
        return planned, Simulator(planned).run()
    except (SimulationCapacityError, SimulationError):
        return None, None


def repair_stalls(plan: SpanPlan, log, cap: int | None, work: float | None) -> bool:
    """Open the spans of the operands that tasks waited for earlier, or merge them with the span before.  True if changed."""
    index = {t.id: i for i, t in enumerate(plan.chain.tasks)}
    changed = False
    for tid, (missing, _short) in sorted(log.stall_causes.items(), key=lambda kv: -log.stalls.get(kv[0], 0.0)):
        if log.stalls.get(tid, 0.0) <= 0.0 or tid not in index:
            continue
        u = index[tid]
        for o in missing:
            k = plan.span_of(o, u)
            if k is None or k == 0 and plan.pinned_start[o]:
                continue
            a, b = plan.spans[o][k]
            size = plan.facts[o].size
            floor = plan.spans[o][k - 1][1] + 1 if k > 0 else plan.first_legal[o]
            # twice the lead, measured on the stall-free clock, but no further than the level allows
            lead = max(plan.cum[u] - plan.cum[a], plan.tau_in(o))
            want = int(np.searchsorted(plan.cum, plan.cum[u] - 2.0 * lead, side="right")) - 1
            want = max(want, floor, 0)
            new_a = a
            while new_a > want and (work is None or plan.level[new_a - 1] + size <= work):
                new_a -= 1
            if new_a <= floor and k > 0:
                new_a = floor                                   # reached the span before: the two merge, the round trip is gone
            if new_a < a:
                plan.add(o, new_a, a - 1)
                changed = True
    return changed


def min_grow(chain: TaskChain, fast_memory_capacity: int | None = None, beam: int = 3, rounds: int = 4) -> TaskChain:
    cap = fast_memory_capacity if fast_memory_capacity is not None else chain.fast_memory_capacity
    base = chain.bare()
    check_input(base, cap, "min_grow")
    grid = [GrowKnobs(h, s, p) for p in ("time", "tasks") for h in (0.0, 0.03, 0.08, 0.15) for s in (1.0, 1.5, 2.5)]
    if cap is None:
        grid = [GrowKnobs(0.0, 1.5, "time")]
    pool = []                                                    # (makespan, plan, planned chain, knobs)
    seen = set()
    first_error = None
    for knobs in grid:
        try:
            plan = grow_static(base, cap, knobs)
        except PlanningError as e:
            first_error = first_error or e
            if "least residency" in str(e):
                raise
            continue
        sig = hash(tuple((o, tuple(map(tuple, s))) for o, s in sorted(plan.spans.items())))
        if sig in seen:
            continue
        seen.add(sig)
        planned, log = _simulate(plan, cap)
        if planned is not None:
            pool.append((log.makespan, plan, planned, log, knobs))
    if not pool:
        raise PlanningError(f"min_grow: no grown plan completes under {cap} bytes ({first_error})")
    pool.sort(key=lambda x: x[0])
    pool = pool[:beam]
    for _ in range(rounds):
        nxt = list(pool)
        improved = False
        for ms, plan, planned, log, knobs in pool:
            if not log.stalls:
                continue
            trial = plan.copy()
            work = None if cap is None else cap * (1.0 - knobs.headroom)
            if not repair_stalls(trial, log, cap, work):
                continue
            p2, l2 = _simulate(trial, cap)
            if p2 is not None and l2.makespan < ms - 1e-9:
                nxt.append((l2.makespan, trial, p2, l2, knobs))
                improved = True
        nxt.sort(key=lambda x: x[0])
        pool = nxt[:beam]
        if not improved:
            break
    return pool[0][2]
