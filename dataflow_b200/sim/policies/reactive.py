"""belady_reactive: Belady's rule applied late, on a shadow run.

The planner steps a ``Shadow`` through the chain and decides each boundary from the state it finds there, never ahead of
need:

    deaths        what the task just used for the last time is released (offloaded when it must end in backing memory and
                  the fast copy is the only current one).
    fetches       an absent operand is fetched only when waiting one more boundary would make it late: the lane's clear
                  time plus its transfer time no longer fits before the start of the task that reads it (estimated from the
                  current time and the runtimes in between).  Operands of the very next task are always fetched.
    evictions     only when the next task, plus what has been asked of the ``from_slow`` lane, does not fit: the resident
                  whose next use lies farthest in the future goes first (Belady), a release when a current backing copy
                  exists, an offload otherwise.  Operands of the next task are never victims.
    probe         before the boundary is closed a fork of the shadow runs the next task; if it cannot start (nothing in
                  flight and not enough room) more victims are taken, and only when none are left does planning fail.

No portfolio, no tuning, one pass.
Reference role: ``src/dataflow_sim/policies/belady_reactive.py`` (a forward walk that queries and mutates a shadow).
"""
from __future__ import annotations


from ..errors import SimulationCapacityError, SimulationError
from ..schema import TaskChain
from .pressurefit import PlanningError
from .shadow import Shadow
from .spans import check_input

INF = float("inf")


class _Future:
    """Who reads what, and when next."""

    def __init__(self, chain: TaskChain):
        self.uses: dict[str, list[int]] = {}
        n = len(chain.tasks)
        for i, t in enumerate(chain.tasks):
            for o in t.inputs:
                self.uses.setdefault(o, []).append(i)
        for o, loc in chain.final_locations.items():
            if loc == "fast":
                self.uses.setdefault(o, []).append(n)
        self.ptr = {o: 0 for o in self.uses}

    def next_use(self, o: str, after: int) -> int | None:
        us = self.uses.get(o)
        if not us:
            return None
        p = self.ptr[o]
        while p < len(us) and us[p] <= after:
            p += 1
        self.ptr[o] = p
        return us[p] if p < len(us) else None


def belady_reactive(chain: TaskChain, fast_memory_capacity: int | None = None, horizon: int = 64, slack: float = 1.1) -> TaskChain:
    cap = fast_memory_capacity if fast_memory_capacity is not None else chain.fast_memory_capacity
    base = chain.bare()
    check_input(base, cap, "belady_reactive")
    tasks = base.tasks
    n = len(tasks)
    fut = _Future(base)
    final = base.final_locations
    sizes = base.sizes()
    try:
        sh = Shadow(base, cap)
        # operands of the first task start in fast memory when they only exist in backing memory: there is no boundary before it
        if n:
            first = [o for o in tasks[0].inputs if sh.where(o)[0] is None]
            if first:
                from ..schema import Object
                extra = [Object(o, sizes[o], "fast", sh.pool[(o, "backing")].type) for o in first]
                sh = Shadow(base, cap, initial=list(base.initial_memory) + extra)
        while not sh.done:
            task = sh.step()
            i = sh.idx
            asked: set[str] = set(sh.queued("from_slow"))
            fl = sh.flight["from_slow"]
            if fl is not None:
                asked.add(fl.obj)
            leaving: set[str] = set()
            if i == 0:
                # initial fast objects nothing ever reads leave at the first boundary
                for o, e in list(sh.resident().items()):
                    if o not in fut.uses and final.get(o) != "fast" and o not in task.inputs:
                        (sh.offload if final.get(o) == "backing" and sh.needs_offload(o) else sh.release)(o)
                        leaving.add(o)
            # deaths
            for o in dict.fromkeys(list(task.inputs) + [x.id for x in task.outputs if x.location == "fast"]):
                if fut.next_use(o, i) is not None or sh.where(o)[0] != "live":
                    continue
                if final.get(o) == "fast":
                    continue
                if final.get(o) == "backing" and sh.needs_offload(o):
                    sh.offload(o)
                else:
                    sh.release(o)
                leaving.add(o)
            nxt = tasks[i + 1] if i + 1 < n else None
            need = 0 if nxt is None else nxt.workspace_bytes + sum(x.size for x in nxt.outputs if x.location == "fast")
            outgoing = sum(x.size for x in sh.queue["to_slow"]) + (sh.flight["to_slow"].size if sh.flight["to_slow"] else 0)
            held = sh.fast_used - sum(sizes[o] for o in leaving) - outgoing + sum(x.size for x in sh.queue["from_slow"]) \
                + sum(x.size for xs in sh.deferred.values() for x in xs)
            # fetches, in need order: only what is about to be late, and (beyond the next task) only while it fits beside
            # what is here, so that the head of the FIFO lane is always the operand needed first and always finds room
            t_need = sh.now
            lane = sh.lane_clear("from_slow")
            last_asked_need = i + 1
            full = False
            for j in range(i + 1, min(i + 1 + horizon, n)):
                for o in tasks[j].inputs:
                    if o in asked or o in leaving:
                        continue
                    fs, bs = sh.where(o)
                    if fs in ("live", "inbound", "reserved") or (fs is None and bs is None):
                        continue                       # resident or arriving, or not produced yet
                    # (a copy on its way out is asked back: the fetch waits for the offload to complete)
                    tau = sh.fetch_time(o)
                    nxt_boundary = sh.now + tasks[i + 1].runtime
                    late_if_we_wait = max(lane, nxt_boundary) + tau * slack > t_need
                    fits = cap is None or held + sizes[o] + need <= cap
                    if j == i + 1 or (late_if_we_wait and fits):
                        sh.prefetch(o)
                        asked.add(o)
                        lane = max(lane, sh.now) + tau
                        held += sizes[o]
                        last_asked_need = j
                    elif late_if_we_wait:
                        full = True
                        break
                if full:
                    break
                t_need += tasks[j].runtime
            # evictions: only when the next task and what the lane will bring do not fit.  A victim is needed later than
            # everything that has been asked for (an earlier need sent away now would queue behind later ones)
            if cap is not None and nxt is not None:
                keep = set(nxt.inputs)
                pending_need = max([last_asked_need] + [fut.next_use(o, i) or 0 for o in sh.queued("from_slow")])
                over = held + need - cap
                ranked = sorted(((fut.next_use(o, i) or INF, e.size, o) for o, e in sh.resident().items()
                                 if o not in keep and o not in leaving and e.size > 0), reverse=True)
                victims = [v for v in ranked if v[0] > pending_need]
                last_resort = [v for v in ranked if v[0] <= pending_need]       # only when the next task cannot start otherwise
                k = 0
                while over > 0 and k < len(victims):
                    _, size, o = victims[k]
                    k += 1
                    (sh.offload if sh.needs_offload(o) else sh.release)(o)
                    leaving.add(o)
                    over -= size
                # probe: can the next task start at all?
                victims = victims + last_resort
                for _ in range(len(victims) + 1):
                    stall, err = sh.lookahead(1)
                    if err is None:
                        break
                    if not isinstance(err, SimulationCapacityError) or k >= len(victims):
                        raise err
                    _, size, o = victims[k]
                    k += 1
                    (sh.offload if sh.needs_offload(o) else sh.release)(o)
                    leaving.add(o)
            sh.commit()
        planned, _log = sh.result()
    except (SimulationCapacityError, SimulationError) as e:
        raise PlanningError(f"belady_reactive: {e}") from None
    return planned
