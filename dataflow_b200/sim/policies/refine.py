"""Lead-time refinement of a finished plan: fire late fetches earlier, keep the change when the simulator says it helped.

Works on any annotated chain, whichever planner wrote it.  A verified run names, for every task that waited, the operands
that were not yet live when it first blocked.  For each of those the fetch that brings the operand in (the last
``prefetch_after`` of it before the task) is moved to an earlier task: far enough to double its lead on the stall-free
clock, never before the task that last touched the object (the one that read, produced, released or offloaded it; a fetch
on the very task that offloads is allowed, it waits for the offload).  The moved plan is simulated; it replaces the
current one when it completes under the capacity with a smaller makespan.  When moving every late fetch at once does not
help (earlier fetches hold memory longer and can push something else out of time), only the fetch behind the longest wait
is moved.  A few rounds, until nothing improves.
Reference role: ``src/dataflow_sim/policies/pressurefit_aux/residency_refinement.py`` (lead-time requests on a finished
residency plan).
"""
from __future__ import annotations

from dataclasses import replace

import numpy as np

from ..errors import SimulationCapacityError, SimulationError
from ..schema import EventLog, TaskChain, TransferTrigger
from ..simulator import Simulator, transfer_runtime


def _late_fetches(chain: TaskChain, log: EventLog) -> list[tuple[float, int, str]]:
    """(microseconds waited, index of the waiting task, operand) for every operand a task waited for, longest wait first."""
    index = {t.id: i for i, t in enumerate(chain.tasks)}
    out = []
    for tid, (missing, _short) in log.stall_causes.items():
        w = log.stalls.get(tid, 0.0)
        if w > 0 and tid in index:
            out.extend((w, index[tid], o) for o in missing)
    out.sort(reverse=True)
    return out


def _move_earlier(chain: TaskChain, moves: list[tuple[float, int, str]], factor: float) -> TaskChain | None:
    tasks = chain.tasks
    cum = np.concatenate([[0.0], np.cumsum([t.runtime for t in tasks])])
    sizes = chain.sizes()
    pre = {i: list(t.prefetch_after) for i, t in enumerate(tasks)}
    changed = False
    for _w, u, o in moves:
        k = next((j for j in range(u - 1, -1, -1) if any(tr.obj_id == o for tr in pre[j])), None)
        if k is None:
            continue
        # the latest task before the fetch that has anything to do with the object
        floor = 0
        for j in range(k - 1, -1, -1):
            t = tasks[j]
            if o in t.inputs or o in t.releases_after or any(x.id == o for x in t.outputs) \
                    or any(tr.obj_id == o for tr in t.offload_after) or any(tr.obj_id == o for tr in pre[j]):
                floor = j
                break
        tau = transfer_runtime(sizes[o], chain.bandwidth_from_slow, None, "from_slow") if chain.bandwidth_from_slow else 0.0
        lead = max(cum[u] - cum[k + 1], tau)
        want = int(np.searchsorted(cum, cum[u] - factor * lead, side="right")) - 2     # fire after the task that ends by then
        new_k = max(want, floor)
        if new_k >= k:
            continue
        trig = next(tr for tr in pre[k] if tr.obj_id == o)
        pre[k].remove(trig)
        pre[new_k].append(TransferTrigger(o, trig.runtime))
        changed = True
    if not changed:
        return None
    return replace(chain, tasks=[replace(t, prefetch_after=pre[i]) for i, t in enumerate(tasks)])


def refine_leads(chain: TaskChain, log: EventLog | None = None, rounds: int = 3, factor: float = 2.0):
    """Returns ``(chain, log, accepted_moves)``; the chain is the input when nothing helped."""
    cap = chain.fast_memory_capacity
    if log is None:
        log = Simulator(chain).run()
    accepted = 0
    for _ in range(rounds):
        late = _late_fetches(chain, log)
        if not late:
            break
        better = None
        for batch in (late, late[:1]):
            trial = _move_earlier(chain, batch, factor)
            if trial is None:
                continue
            try:
                tl = Simulator(trial).run()
            except (SimulationCapacityError, SimulationError):
                continue
            if tl.makespan < log.makespan - 1e-9 and (cap is None or tl.peak_fast_memory_bytes <= cap):
                better = (trial, tl, len(batch))
                break
        if better is None:
            break
        chain, log = better[0], better[1]
        accepted += better[2]
    return chain, log, accepted
