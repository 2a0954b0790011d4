"""max_reduce: start with everything resident and take residency away where the accounting says it does not fit.

Pure memory accounting: no lane clocks, no simulator inside the loop.  The plan starts as ``SpanPlan.fill_max`` (every
object in fast memory from the first moment it may exist to its last touch).  While some task's level exceeds the capacity:

    1. take the task ``i`` with the largest excess;
    2. every object that is resident during ``i`` without being touched by it offers one cut: leave after its previous touch,
       come back just in time for its next one (lead = its own transfer time on the stall-free clock).  The cut helps only if
       the bytes are really away during ``i``: an offload keeps its fast copy until it completes, a fetch charges from its
       start.  When no object can be away in time, fetches that arrive late (fired right before the use) are offered instead;
    3. the offer that removes the most excess (summed over all tasks it frees) per microsecond of lane time it costs wins.

When no object offers a cut that frees ``i``, no plan of this shape fits and ``PlanningError`` is raised.  The simulator sees
the result once, at the end (``spans.verify``): lane contention the accounting ignored shows up there as stalls, and as a
smaller effective capacity when bytes in flight push the run over the cap.
Reference role: ``src/dataflow_sim/policies/max_reduce.py`` (residency by accounting, then triggers).
"""
from __future__ import annotations


import numpy as np

from ..schema import TaskChain
from .pressurefit import PlanningError
from .spans import SpanPlan, check_input, verify


def reduce_to_fit(plan: SpanPlan, cap: float, slack: float = 1.0) -> int:
    """Cut spans until ``plan.level <= cap`` everywhere; returns the number of cuts."""
    cuts = 0
    n = plan.n
    names = [o for o in plan.spans if plan.facts[o].size > 0 and plan.spans[o]]
    cover = np.zeros((len(names), n), dtype=bool)                        # cover[k, i]: object k is resident during task i
    for k, o in enumerate(names):
        for a, b in plan.spans[o]:
            cover[k, a:b + 1] = True
    touched = [set(plan.touch[o]) for o in names]
    rounds = 0
    while n:
        over = plan.level - cap
        i = int(np.argmax(over))
        if over[i] <= 0:
            return cuts
        rounds += 1
        if rounds > 4 * n + 64:
            raise PlanningError("max_reduce: the reduction does not converge")
        pos = np.maximum(over, 0.0)
        excess = np.concatenate([[0.0], np.cumsum(pos)])                 # excess[j]: positive excess summed over tasks < j
        hot = np.concatenate([[0], np.cumsum(pos > 0)])
        offers = []
        for timely in (True, False):
            for k in np.nonzero(cover[:, i])[0]:
                if i in touched[k]:
                    continue
                o = names[k]
                before, after = plan.neighbours(o, i)
                if after is None:
                    continue
                # an initial backing object waiting for its first touch (no touch before): bring it later, not up front
                lo = 0 if before is None else (plan.first_free_after(o, before) if timely else before + 1)
                hi = (plan.lead_start(o, after, slack) if timely else after) - 1
                if not (lo <= i <= hi):
                    continue                                             # the bytes would not really be away during task i
                size = plan.facts[o].size
                relief = min(excess[hi + 1] - excess[lo], size * float(hot[hi + 1] - hot[lo]))
                cost = plan.tau_in(o) + (0.0 if before is None or plan.clean_until(o, before) else plan.tau_out(o))
                offers.append((relief / max(cost, 1e-9), size, int(k), 0 if before is None else before + 1, hi))
            if offers:
                break               # late fetches (the task after waits for its operand) only when nothing timely frees task i
        if not offers:
            held = sorted(((plan.facts[o].size, o) for o in names if i in plan.touch[o]), reverse=True)[:4]
            raise PlanningError(f"max_reduce: task {plan.chain.tasks[i].id!r} holds {plan.level[i]:.0f} bytes against {cap:.0f} and "
                                f"nothing resident can be away during it (largest operands: {held})")
        offers.sort(reverse=True)
        for _, _, k, lo, hi in offers:                                    # the best offers first, until this task fits
            plan.cut(names[k], lo, hi)
            cover[k, lo:hi + 1] = False
            cuts += 1
            if plan.level[i] <= cap:
                break
    return cuts


def max_reduce(chain: TaskChain, fast_memory_capacity: int | None = None, slack: float = 1.0) -> TaskChain:
    cap = fast_memory_capacity if fast_memory_capacity is not None else chain.fast_memory_capacity
    base = chain.bare()
    check_input(base, cap, "max_reduce")

    def build(cap_eff):
        plan = SpanPlan(base).fill_max(slack=slack)
        if cap_eff is not None:
            reduce_to_fit(plan, float(cap_eff), slack)
        return plan.emit(cap)

    return verify(build, cap, "max_reduce")[0]
