"""sliding_window: the hand pattern, with no knowledge of the capacity.

Every object is kept in fast memory for a window of ``window_size`` tasks around each of its touches and lives in backing
memory in between: after a touch it stays for the window (a touch that follows within two windows keeps it resident),
then leaves; it is fetched back ``window_size`` tasks before the next touch.  Objects that start in backing memory arrive
``window_size`` tasks before their first touch (or are placed up front when that is before the first task).  This is what
one writes by hand for a layered model - "keep two layers of weights ahead, send activations away after the forward pass,
bring them back two layers before their backward pass" - stated over tasks instead of layer names, so it applies to any
chain.

The pattern does not look at the capacity: the simulator decides whether the result fits.  When it does not, smaller
windows are tried down to one task, and ``PlanningError`` is raised when even that does not fit.
Reference role: ``src/dataflow_sim/policies/sliding_window.py`` (a fixed release / prefetch pattern with a window size).
"""
from __future__ import annotations


from ..errors import SimulationCapacityError, SimulationError
from ..schema import TaskChain
from ..simulator import Simulator
from .pressurefit import PlanningError
from .spans import SpanPlan, check_input


def window_plan(chain: TaskChain, window: int) -> SpanPlan:
    plan = SpanPlan(chain)
    for o, touches in plan.touch.items():
        if not touches:
            continue
        for j, u in enumerate(touches):
            if j == 0 and plan.pinned_start[o]:
                a = u
            else:
                floor = touches[j - 1] + 1 if j > 0 else plan.first_legal[o]
                a = max(u - window, floor, 0)
            last = j == len(touches) - 1
            b = u if last else min(u + window, touches[j + 1] - 1)
            plan.add(o, a, b)
    return plan


def sliding_window(chain: TaskChain, fast_memory_capacity: int | None = None, window_size: int = 2) -> TaskChain:
    if window_size < 1:
        raise ValueError("window_size must be at least 1")
    cap = fast_memory_capacity if fast_memory_capacity is not None else chain.fast_memory_capacity
    base = chain.bare()
    check_input(base, cap, "sliding_window")
    err = None
    for w in range(window_size, 0, -1):
        planned = window_plan(base, w).emit(cap)
        try:
            Simulator(planned).run()
            return planned
        except (SimulationCapacityError, SimulationError) as e:
            err = err or e
    # the window before a touch is what the pattern is about; the one after it is a convenience that can go
    plan = SpanPlan(base).fill_min(0.0)
    planned = plan.emit(cap)
    try:
        Simulator(planned).run()
        return planned
    except (SimulationCapacityError, SimulationError):
        raise PlanningError(f"sliding_window: no window from {window_size} down to 0 tasks fits {cap} bytes ({err})") from None
