"""Lookahead — a planner that decides directives *while the simulator runs*.

PressureFit lays residency out on a stall-free timeline and checks it afterwards; when the two
copy lanes are the bottleneck (large optimizer state streaming through a small fast tier) the
real timeline drifts away from that layout and most candidates have to be repaired or fail.
This planner instead sits inside the event-driven simulator: at every task boundary it sees the
true state of the run (time, resident set, dirty bits, lane queues) together with complete
knowledge of the future of the chain, and fills in that task's ``releases_after``,
``offload_after`` and ``prefetch_after``.  The run that produced the decisions IS the
verification: the annotated chain replays to the same event log.

Decisions at the boundary after task ``i`` (time ``t``):

* **Deaths.**  Objects whose last use was ``i`` are released, or offloaded when their terminal
  location is the backing tier and the fast copy is the only current one.
* **Must-start prefetches.**  Absent objects are ordered by the task that needs them; a backward
  pass over the ``from_slow`` lane (need time, transfer time × slack, FIFO order) gives each its
  latest start.  Those whose latest start falls before the next boundary are issued now.
* **Free-room prefetches.**  Further absent objects are issued early, in need order, while the
  lane is short of work and the projected residency has room for them from now until their use.
* **Evictions.**  The projected residency (what is resident, what is born, what dies, what must
  be reloaded, task by task) is scanned ahead; at the first task that would not fit, residents
  that are not needed before it are evicted — a release when a valid backing copy exists, an
  offload otherwise — ranked by the victim score, as soon as the time left is no more than
  ``evict_lead`` × the time the ``to_slow`` lane needs to free the deficit.

The reference has no counterpart of this file; its planners are offline
(``src/dataflow_sim/policies/*.py``).
"""
from __future__ import annotations

import bisect
from dataclasses import dataclass, replace
from typing import Callable, Sequence

import numpy as np

from ..errors import SimulationCapacityError, SimulationError
from ..schema import Object, Task, TaskChain, TransferTrigger
from ..simulator import BACKING, FAST, Simulator, compute_lower_bound, transfer_runtime
from ..validate import validate_planning_input


# victim score(size, seconds-to-next-use in µs, needs_offload, type) -> larger is evicted first
def _v_farthest(size, dist, needs_offload, typ):
    return dist


def _v_cost_aware(size, dist, needs_offload, typ):
    return dist * (0.5 if needs_offload else 1.0)


def _v_clean_first(size, dist, needs_offload, typ):
    return (0.0 if needs_offload else 1e15) + dist


def _v_bytes(size, dist, needs_offload, typ):
    return dist * float(size) ** 0.5 * (0.5 if needs_offload else 1.0)


@dataclass(frozen=True)
class LookaheadSpec:
    name: str
    victim: Callable[[int, float, bool, str], float]
    slack: float = 1.25          # transfer-time multiplier of the must-start pass
    evict_lead: float = 2.0      # evict when time left <= evict_lead x time to free the deficit
    early_room: float = 1.0      # fraction of the spare room free-room prefetches may take (0 = none)


LOOKAHEAD_SPECS: tuple[LookaheadSpec, ...] = (
    LookaheadSpec("cost_aware", _v_cost_aware),
    LookaheadSpec("farthest", _v_farthest),
    LookaheadSpec("clean_first", _v_clean_first),
    LookaheadSpec("cost_aware_tight", _v_cost_aware, 1.0, 1.25),
    LookaheadSpec("cost_aware_wide", _v_cost_aware, 1.6, 3.0),
    LookaheadSpec("bytes", _v_bytes),
    LookaheadSpec("cost_aware_lazy", _v_cost_aware, 1.25, 2.0, 0.0),
)


class _Planner(Simulator):
    """The simulator with the oracle in the loop.  Works on a private copy of the chain's tasks."""

    WINDOW = 512           # tasks scanned ahead for residency violations
    MUST_START_DEPTH = 160  # absent objects considered by the backward pass

    def __init__(self, chain: TaskChain, spec: LookaheadSpec, headroom: float):
        super().__init__(chain)
        self.spec = spec
        tasks = chain.tasks
        n = self.n = len(tasks)
        self.rt = np.array([t.runtime for t in tasks] + [0.0], dtype=np.float64)
        self.cum = np.concatenate([[0.0], np.cumsum(self.rt)])            # stall-free start of task j
        self.ws = np.array([t.workspace_bytes for t in tasks] + [0, 0], dtype=np.float64)
        self.bw_in, self.bw_out = chain.bandwidth_from_slow, chain.bandwidth_to_slow
        cap = chain.fast_memory_capacity
        self.cap_eff = None if cap is None else cap * (1.0 - headroom)
        self.size: dict[str, int] = {}
        self.typ: dict[str, str] = {}
        self.uses: dict[str, list[int]] = {}
        self.ptr: dict[str, int] = {}
        self.delta = np.zeros(n + 3, dtype=np.float64)
        self.absent: list[tuple[int, str]] = []
        self.emergencies = 0
        self.preplaced: list[str] = []
        init_fast, init_back = set(), set()
        for o in chain.initial_memory:
            self.size[o.id], self.typ[o.id] = o.size, o.type
            self.uses.setdefault(o.id, [])
            (init_fast if o.location == FAST else init_back).add(o.id)
        born_fast: dict[str, int] = {}
        born_back: dict[str, int] = {}
        for i, t in enumerate(tasks):
            for out in t.outputs:
                self.size[out.id], self.typ[out.id] = out.size, out.type
                self.uses.setdefault(out.id, [])
                (born_fast if out.location == FAST else born_back)[out.id] = i
            for inp in t.inputs:
                self.uses[inp].append(i)
        for o, loc in chain.final_locations.items():
            if loc == FAST and o in self.uses:
                self.uses[o].append(n)            # must be resident when the chain ends
        self.level = float(sum(self.size[o] for o in init_fast))
        for o, us in self.uses.items():
            self.ptr[o] = 0
            sz = self.size[o]
            birth = born_fast.get(o, born_back.get(o, -1))
            death = (us[-1] if us else max(birth, -1)) + 1
            if o in init_fast:
                self.delta[min(death, n + 1)] -= sz
            elif o in born_fast:
                self.delta[born_fast[o]] += sz
                self.delta[min(death, n + 1)] -= sz
            elif us:                                # lives in backing until its first use
                self.delta[us[0]] += sz
                self.delta[min(death, n + 1)] -= sz
                if o in init_back:
                    bisect.insort(self.absent, (us[0], o))
        self.born_back = born_back
        self._preplace()
        self.level += float(self.delta[0])          # residency during task 0

    def _preplace(self) -> None:
        """Objects that no prefetch issued after task 0 could deliver in time start in fast memory
        (as far as the projected residency has room for them)."""
        if not self.absent or self.n == 0:
            return
        head = self.absent[:self.MUST_START_DEPTH]
        lim = float("inf")
        ls = [0.0] * len(head)
        for i in range(len(head) - 1, -1, -1):
            u, o = head[i]
            lim = min(float(self.cum[min(u, self.n)]), lim) - self._dur_in(o) * self.spec.slack
            ls[i] = lim
        hi = min(self.WINDOW, self.n + 1)
        proj = None if self.cap_eff is None else self.level + np.cumsum(self.delta[0:hi]) + self.ws[0:hi]
        k = 0
        while k < len(head) and ls[k] <= float(self.rt[0]):
            u, o = head[k]
            sz = self.size[o]
            if proj is not None and u > 0:
                end = min(max(u, 1), len(proj))
                if float(proj[:end].max()) + sz > self.cap_eff:
                    break
                proj[:min(u, hi)] += sz
            self.chain.initial_memory.append(Object(o, sz, FAST, self.typ[o]))
            self.preplaced.append(o)
            self.level += sz
            self.delta[u] -= sz
            k += 1
        del self.absent[:k]

    # ---- helpers
    def _dur_in(self, o: str) -> float:
        return transfer_runtime(self.size[o], self.bw_in, None, "from_slow")

    def _dur_out(self, o: str) -> float:
        return transfer_runtime(self.size[o], self.bw_out, None, "to_slow")

    def _backlog(self, direction: str, now: float) -> float:
        b = 0.0
        f = self.flight[direction]
        if f is not None:
            b += max(f.end - now, 0.0)
        for x in self.queue[direction]:
            b += x.runtime
        if direction == "from_slow":
            for lst in self.deferred.values():
                for x in lst:
                    b += x.runtime
        return b

    def _next_use(self, o: str) -> int | None:
        us, p = self.uses[o], self.ptr[o]
        return us[p] if p < len(us) else None

    def _needs_offload(self, o: str) -> bool:
        e = self.pool[(o, FAST)]
        b = self.pool.get((o, BACKING))
        return e.dirty or b is None or b.state != "live"

    # ---- decisions
    def _issue_prefetch(self, task: Task, o: str, need: int, idx: int) -> None:
        task.prefetch_after.append(TransferTrigger(o))
        sz = self.size[o]
        self.delta[idx + 1] += sz
        self.delta[need] -= sz

    def _prefetch_pass(self, idx: int, task: Task, t: float) -> None:
        if not self.absent:
            return
        spec = self.spec
        nxt = idx + 1
        rt_next = float(self.rt[nxt]) if nxt <= self.n else 0.0
        head = self.absent[:self.MUST_START_DEPTH]
        k = len(head)
        need_t = [t + float(self.cum[min(u, self.n)] - self.cum[min(nxt, self.n)]) for u, _ in head]
        dur = [self._dur_in(o) for _, o in head]
        ls = [0.0] * k
        lim = float("inf")
        for i in range(k - 1, -1, -1):
            lim = min(need_t[i], lim) - dur[i] * spec.slack
            ls[i] = lim
        backlog = self._backlog("from_slow", t)
        out_backlog = None
        hi = min(nxt + self.WINDOW, self.n + 1)
        proj = None if self.cap_eff is None else self.level + np.cumsum(self.delta[nxt:hi]) + self.ws[nxt:hi]
        evicted: set[str] = set(x.obj_id for x in task.offload_after) | set(task.releases_after)
        issued = 0
        while issued < k:
            u, o = head[issued]
            must = ls[issued] <= t + rt_next          # waiting for the next boundary would make it late
            if not must and (spec.early_room <= 0 or backlog >= 2.0 * rt_next + dur[issued]):
                break
            sz = self.size[o]
            if proj is not None and len(proj):
                end = min(max(u - nxt, 1), len(proj))
                peak = float(proj[:end].max())
                room = self.cap_eff - peak if must else (self.cap_eff - peak) * spec.early_room
                if sz > room:
                    if not must:
                        break
                    # make room only at the expense of residents needed LATER than this object
                    cands = self._victims(idx, u, evicted)
                    deficit = sz - room
                    if sum(self.size[c[1]] for c in cands) < deficit:
                        break
                    if out_backlog is None:
                        out_backlog = self._backlog("to_slow", t)
                    for _, vo, vu, voff in cands:
                        if deficit <= 0:
                            break
                        evicted.add(vo)
                        out_backlog = self._evict(task, vo, vu, voff, idx, nxt, t, out_backlog)
                        proj[:max(min(vu, hi) - nxt, 0)] -= self.size[vo]
                        deficit -= self.size[vo]
                proj[:max(min(u, hi) - nxt, 0)] += sz
            self._issue_prefetch(task, o, u, idx)
            backlog += dur[issued]
            issued += 1
        if issued:
            issued_set = {o for _, o in head[:issued]}
            self.absent = [e for e in self.absent if e[1] not in issued_set]

    def _victims(self, idx: int, before: int, exclude: set[str]) -> list[tuple[float, str, int, bool]]:
        """Residents not needed before task ``before``: (score, id, next use, needs offload), best first."""
        out = []
        nxt = min(idx + 1, self.n)
        for (o, loc), e in self.pool.items():
            if loc != FAST or e.state != "live" or o in exclude:
                continue
            u = self._next_use(o)
            if u is None or u <= before:
                continue
            off = self._needs_offload(o)
            dist = float(self.cum[min(u, self.n)] - self.cum[nxt])
            out.append((self.spec.victim(e.size, dist, off, e.type), o, u, off))
        out.sort(key=lambda x: -x[0])
        return out

    def _evict(self, task: Task, o: str, u: int, off: bool, idx: int, j1: int, t: float, out_backlog: float) -> float:
        sz = self.size[o]
        nxt = idx + 1
        if off:
            task.offload_after.append(TransferTrigger(o))
            d = self._dur_out(o)
            free_t = float(self.cum[min(nxt, self.n)]) + out_backlog + d
            jf = int(np.searchsorted(self.cum, free_t, side="left"))
            jf = max(nxt, min(jf, max(j1, nxt)))
            out_backlog += d
        else:
            task.releases_after.append(o)
            jf = nxt
        self.delta[jf] -= sz
        self.delta[u] += sz
        bisect.insort(self.absent, (u, o))
        return out_backlog

    def _evict_pass(self, idx: int, task: Task, t: float) -> None:
        if self.cap_eff is None:
            return
        nxt = idx + 1
        if nxt > self.n:
            return
        hi = min(nxt + self.WINDOW, self.n + 1)
        rt_next = float(self.rt[nxt])
        out_backlog = self._backlog("to_slow", t)
        evicted: set[str] = set(x.obj_id for x in task.offload_after) | set(task.releases_after)
        avail = self.cum[nxt:hi] - self.cum[nxt]
        for _ in range(4096):
            proj = self.level + np.cumsum(self.delta[nxt:hi]) + self.ws[nxt:hi]
            over = proj - self.cap_eff
            bad = np.nonzero(over > 0)[0]
            if bad.size == 0:
                return
            t_req = out_backlog + over[bad] / float(self.bw_out or 1)
            urgent = avail[bad] <= self.spec.evict_lead * t_req + rt_next
            if not urgent.any():
                return
            j1 = nxt + int(bad[0])
            cands = self._victims(idx, j1, evicted)
            if not cands:
                return          # nothing resident is idle through the violation; objects born later will be
            _, o, u, off = cands[0]
            evicted.add(o)
            out_backlog = self._evict(task, o, u, off, idx, j1, t, out_backlog)

    def _before_directives(self, idx: int, task: Task, t: float) -> None:
        nxt = idx + 1
        # pointers past this task; objects born in backing become absent
        for o in task.inputs:
            us, p = self.uses[o], self.ptr[o]
            while p < len(us) and us[p] <= idx:
                p += 1
            self.ptr[o] = p
        for out in task.outputs:
            if out.location == BACKING and self.uses[out.id]:
                bisect.insort(self.absent, (self.uses[out.id][0], out.id))
        # deaths
        for o in dict.fromkeys(list(task.inputs) + [x.id for x in task.outputs]):
            if self._next_use(o) is not None:
                continue
            e = self.pool.get((o, FAST))
            if e is None or e.state != "live":
                continue
            if self.chain.final_locations.get(o) == BACKING and self._needs_offload(o):
                task.offload_after.append(TransferTrigger(o))
            else:
                task.releases_after.append(o)
        self._prefetch_pass(idx, task, t)
        self._evict_pass(idx, task, t)
        self.level += float(self.delta[nxt]) if nxt <= self.n + 1 else 0.0

    def _on_deadlock(self, idx: int, task: Task, now: float, need: int, missing: list[str]) -> bool:
        """Nothing in flight and the task cannot start: amend the previous task's directives."""
        if idx == 0:
            return False
        prev = self.chain.tasks[idx - 1]
        self.emergencies += 1
        if self.emergencies > 4 * self.n:
            return False
        progress = False
        for o in missing:
            e = self.pool.get((o, FAST))
            b = self.pool.get((o, BACKING))
            if e is None and b is not None and b.state == "live" and all(x.obj_id != o for x in prev.prefetch_after):
                if (self._next_use(o) or idx, o) in self.absent:
                    self.absent.remove((self._next_use(o) or idx, o))
                prev.prefetch_after.append(TransferTrigger(o))
                self.queue["from_slow"].append(_mk_xfer(self, o, "from_slow"))
                progress = True
        cap = self.cap[FAST]
        short = 0 if cap is None else self.used[FAST] + need + sum(
            self.size[o] for o in missing if self.pool.get((o, FAST)) is None) - cap
        if short > 0:
            keep = set(task.inputs)
            for _, o, u, off in self._victims(idx - 1, idx, keep):
                if short <= 0:
                    break
                e = self.pool[(o, FAST)]
                if off:
                    prev.offload_after.append(TransferTrigger(o))
                    e.state = "pending_outbound"
                    self.queue["to_slow"].append(_mk_xfer(self, o, "to_slow"))
                else:
                    prev.releases_after.append(o)
                    self.used[FAST] -= e.size
                    del self.pool[(o, FAST)]
                bisect.insort(self.absent, (u, o))
                self.delta[u] += self.size[o]
                self.level -= self.size[o]
                short -= e.size
                progress = True
        if progress:
            self._poke(now)
        return progress


def _mk_xfer(sim: "_Planner", o: str, direction: str):
    from ..simulator import _Xfer
    bw = sim.bw_in if direction == "from_slow" else sim.bw_out
    return _Xfer(o, direction, sim.size[o], transfer_runtime(sim.size[o], bw, None, direction), sim.typ[o])


# --------------------------------------------------------------------------- driver
@dataclass
class LookaheadCandidate:
    spec: str
    makespan: float | None
    peak_fast: int | None
    emergencies: int = 0
    error: str | None = None


@dataclass
class LookaheadResult:
    chain: TaskChain
    makespan: float
    peak_fast_bytes: int
    lower_bound: float
    chosen: LookaheadCandidate
    candidates: list[LookaheadCandidate]

    @property
    def idle_fraction(self) -> float:
        return 0.0 if self.makespan <= 0 else 1.0 - self.lower_bound / self.makespan


def _fresh(chain: TaskChain, cap: int | None) -> TaskChain:
    tasks = [replace(t, releases_after=[], offload_after=[], prefetch_after=[]) for t in chain.tasks]
    return replace(chain, tasks=tasks, initial_memory=list(chain.initial_memory), fast_memory_capacity=cap)


def plan_one(chain: TaskChain, cap: int | None, spec: LookaheadSpec, headroom: float = 0.02):
    """One oracle-in-the-loop run; returns (annotated chain, verified event log, emergencies)."""
    work = _fresh(chain, cap)
    sim = _Planner(work, spec, headroom)
    sim.run()
    log = Simulator(work).run()          # replay: emergency amendments move a directive to a task boundary
    return work, log, sim.emergencies


def lookahead(chain: TaskChain, fast_memory_capacity: int | None = None, *,
              specs: Sequence[LookaheadSpec] | None = None, validate: bool = True,
              headrooms: Sequence[float] = (0.02, 0.05), rel_tolerance: float = 1e-9) -> LookaheadResult:
    """Plan ``chain`` under ``fast_memory_capacity``: best verified candidate of the spec portfolio."""
    from .pressurefit import PlanningError
    cap = fast_memory_capacity if fast_memory_capacity is not None else chain.fast_memory_capacity
    base = chain.bare()
    if validate:
        validate_planning_input(base)
    lower = compute_lower_bound(base)
    best = None
    cands: list[LookaheadCandidate] = []
    for spec in (specs or LOOKAHEAD_SPECS):
        for hr in headrooms:
            try:
                planned, log, em = plan_one(base, cap, spec, hr)
            except (SimulationCapacityError, SimulationError) as e:
                cands.append(LookaheadCandidate(f"{spec.name}@{hr}", None, None, 0, str(e)[:300]))
                continue
            c = LookaheadCandidate(f"{spec.name}@{hr}", log.makespan, log.peak_fast_memory_bytes, em)
            cands.append(c)
            if best is None or log.makespan < best[1].makespan - 1e-12:
                best = (planned, log, c)
            if cap is None or log.makespan <= lower * (1 + rel_tolerance) + 1e-9:
                break
        if best is not None and best[1].makespan <= lower * (1 + rel_tolerance) + 1e-9:
            break
    if best is None:
        detail = "; ".join(f"{c.spec}: {c.error}" for c in cands[:3])
        raise PlanningError(f"no lookahead candidate fits {cap} bytes of fast memory ({detail})")
    planned, log, c = best
    return LookaheadResult(planned, log.makespan, log.peak_fast_memory_bytes, lower, c, cands)


def apply_lookahead_policy(chain: TaskChain, fast_memory_capacity: int | None = None, **kw) -> TaskChain:
    return lookahead(chain, fast_memory_capacity, **kw).chain
