"""roundtrip: a constructive planner that books every transfer on a lane timeline before it commits to it.

No simulator inside: the planner works on the stall-free clock with two timelines, one per copy lane, on which transfers
are booked as intervals (one transfer at a time per lane).

    1. placement    initial backing objects are placed in fast memory up front, in order of first use, while the level
                    allows; the rest wait in backing memory.
    2. first fetches   every object that waits in backing memory must be fetched for its first touch.  These are booked
                    backwards from the end of the chain: each takes the latest free interval on ``from_slow`` that ends
                    before its task starts, so later needs never push earlier ones off the lane.
    3. round trips  walk the tasks in order; where the level exceeds the capacity, objects that are resident but idle are
                    sent on a round trip: an offload booked at the earliest free interval of ``to_slow`` after the previous
                    touch, a fetch booked at the latest free interval of ``from_slow`` before the next touch.  A trip is
                    *amortised* when both fit inside the idle gap; amortised trips are preferred, largest bytes x time
                    away first, and a trip is committed only if it actually takes bytes away from the task that needs
                    room.  When amortised trips do not suffice, trips whose fetch arrives late are taken (the next touch
                    will wait for it) rather than giving up.
    4. emit         spans follow from the bookings (a span ends at the previous touch and restarts at the task during which
                    the booked fetch begins).

The simulator sees the result once (``spans.verify``).
Reference role: ``src/dataflow_sim/policies/roundtrip_planner.py`` (mandatory first-use prefetches, then demand-driven round
trips packed on two stream timelines).
"""
from __future__ import annotations


import numpy as np

from ..errors import SimulationError
from ..schema import TaskChain
from .pressurefit import PlanningError
from .spans import LaneTimeline, SpanPlan, check_input, verify


def _task_at(plan: SpanPlan, t: float) -> int:
    """The task during which time ``t`` falls on the stall-free clock (the first task for t <= 0)."""
    return max(int(np.searchsorted(plan.cum, t, side="right")) - 1, 0)


def build_plan(chain: TaskChain, cap: float | None, place_share: float = 0.9) -> SpanPlan:
    plan = SpanPlan(chain)
    n = plan.n
    lane_in, lane_out = LaneTimeline(), LaneTimeline()
    waiting = []                                   # initial backing objects, by first touch
    for o, t in plan.touch.items():
        if not t:
            continue
        f = plan.facts[o]
        if f.birth < 0 and not f.in_fast:
            waiting.append((t[0], o))
        else:
            plan.add(o, min(plan.first_legal[o], t[0]), t[-1])
    waiting.sort()
    # 1. placement by first use while the level allows (the share leaves room for what is born later)
    late = []
    for u, o in waiting:
        t = plan.touch[o]
        size = plan.facts[o].size
        if cap is None or float(plan.level[0:t[-1] + 1].max()) + size <= cap * place_share:
            plan.add(o, 0, t[-1])
        else:
            late.append((u, o))
    # 2. first fetches, booked backwards
    for u, o in sorted(late, reverse=True):
        tau = plan.tau_in(o)
        start = lane_in.latest(float(plan.cum[u]), tau)
        if start is None:
            start = 0.0                              # the lane is full before this task: fetch as early as possible and wait
            start = lane_in.earliest(start, tau)
        lane_in.book(start, tau)
        a = min(_task_at(plan, start), u)
        plan.add(o, max(a, plan.first_legal[o]), plan.touch[o][-1])
    if cap is None:
        return plan
    # 3. round trips where the level exceeds the capacity
    names = [o for o in plan.spans if plan.facts[o].size > 0 and plan.spans[o]]
    cover = np.zeros((len(names), n), dtype=bool)
    for k, o in enumerate(names):
        for a, b in plan.spans[o]:
            cover[k, a:b + 1] = True
    touched = [set(plan.touch[o]) for o in names]
    in_flight = np.zeros(n)                                           # bytes of offloads still holding their fast copy, per task

    def propose(k: int, i: int):
        """The round trip of object ``k`` around task ``i`` as the lanes stand now, or None when it frees nothing there."""
        o = names[k]
        before, after = plan.neighbours(o, i)
        if after is None:
            return None
        clean = before is None or plan.clean_until(o, before)
        t0 = 0.0 if before is None else float(plan.cum[before + 1])
        out_len = 0.0 if clean else plan.tau_out(o)
        out_start = t0 if clean else lane_out.earliest(t0, out_len)
        away_from = out_start + out_len
        tau = plan.tau_in(o)
        in_start = lane_in.latest(float(plan.cum[after]), tau, not_before=away_from)
        amortised = in_start is not None
        if not amortised:
            in_start = lane_in.earliest(max(away_from, float(plan.cum[after]) - tau), tau)
        first = 0 if before is None else before + 1
        lo = first if clean else int(np.searchsorted(plan.cum, away_from, side="left"))
        hi = min(_task_at(plan, in_start), after) - 1
        if not (lo <= i <= hi):
            # the free intervals of the lanes do not leave the bytes away during task i: take the trip anyway, fetched at
            # the last moment, and let the run wait on both ends
            amortised = False
            in_start = lane_in.earliest(max(away_from, float(plan.cum[after]) - tau), tau)
            lo, hi = first, after - 1
            if not (lo <= i <= hi):
                return None
        away = float(plan.cum[hi + 1] - plan.cum[lo])
        return (amortised, plan.facts[o].size * away, k, first, lo, hi, out_start, out_len, in_start, tau)

    for i in range(n):
        scans = 0
        while plan.level[i] > cap:
            scans += 1
            if scans > 8:
                raise PlanningError("roundtrip: the trips do not converge")
            trips = [t for k in np.nonzero(cover[:, i])[0] if i not in touched[k] and (t := propose(int(k), i)) is not None]
            if not trips and plan.level[i] - in_flight[i] <= cap:
                break                                                 # only offloads in flight are in the way: the task waits for them
            if not trips:
                raise PlanningError(f"roundtrip: task {chain.tasks[i].id!r} holds {plan.level[i]:.0f} bytes against {cap:.0f} and "
                                    f"no resident object can take a round trip around it")
            trips.sort(key=lambda x: (x[0], x[1]), reverse=True)
            for stale in trips:                                       # best first; each re-proposed against the lanes as they are now
                t = propose(stale[2], i)
                if t is None:
                    continue
                _, _, k, first, lo, hi, out_start, out_len, in_start, tau = t
                o = names[k]
                if out_len:
                    lane_out.book(out_start, out_len)
                lane_in.book(in_start, tau)
                plan.cut(o, first, hi)
                cover[k, first:hi + 1] = False
                if lo > first:                                        # the offload holds the fast copy until it completes
                    plan.level[first:lo] += plan.facts[o].size
                    in_flight[first:lo] += plan.facts[o].size
                    plan.tails.append((o, first, lo - 1))
                if plan.level[i] <= cap:
                    break
    return plan


def roundtrip_planner(chain: TaskChain, fast_memory_capacity: int | None = None) -> TaskChain:
    cap = fast_memory_capacity if fast_memory_capacity is not None else chain.fast_memory_capacity
    base = chain.bare()
    check_input(base, cap, "roundtrip")
    best = None
    err = None
    for share in (0.9, 0.7, 0.5):
        try:
            planned, log, _ = verify(lambda c: build_plan(base, None if c is None else float(c), share).emit(cap), cap, "roundtrip")
        except (PlanningError, SimulationError) as e:
            err = err or e
            continue
        if best is None or log.makespan < best[1].makespan:
            best = (planned, log)
    if best is None:
        raise PlanningError(str(err))
    return best[0]
