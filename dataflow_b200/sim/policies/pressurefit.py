"""PressureFit — the general planner.

Input: a *bare* TaskChain and a fast-memory capacity.  Output: the same chain
annotated with ``releases_after / offload_after / prefetch_after`` (and initial
placements) such that the simulator completes it under the capacity, chosen as
the fastest of a portfolio of candidates that are each **verified by the
simulator**.  Same contract as the reference's
``src/dataflow_sim/policies/pressurefit.py:147-392`` (5 residency specs × 8
prefetch rules, early exit at the compute-only lower bound); the construction
below is this repository's own:

1. *Facts*: for every object, its birth, ordered uses, mutation points and
   terminal placement.
2. *Residency sweep* (one pass over the stall-free timeline): walk the chain
   keeping a charged-bytes counter; when a task would not fit, evict residents
   that task does not touch, ranked by the residency spec (farthest next use,
   bytes × distance, largest, clean first, role weighted).  An eviction is
   attached to the object's previous use — a release if a valid backing copy
   exists, an offload otherwise — and the object re-enters the counter when its
   just-in-time reload window opens, so reload windows are part of the pressure.
3. *Prefetch rule*: turn reload requests into ``prefetch_after`` anchors on the
   single ``from_slow`` lane (backward just-in-time packing with a slack factor,
   or a fixed task look-ahead); anchors are made monotone in need order so the
   FIFO head is always the earliest-needed object.
4. *Verify* by simulation; on a capacity deadlock shrink the effective cap by the
   reported overage and rebuild (physical repair).
"""
from __future__ import annotations

import heapq
from bisect import bisect_right
from dataclasses import dataclass, field, replace
from typing import Callable, Sequence

from ..errors import SimulationCapacityError, SimulationError
from ..schema import Object, Task, TaskChain, TransferTrigger
from ..simulator import Simulator, compute_lower_bound
from ..validate import validate_planning_input


class PlanningError(RuntimeError):
    """No candidate completed under the capacity."""


# --------------------------------------------------------------------------- facts
@dataclass
class ObjFacts:
    id: str
    size: int
    type: str
    birth: int                      # -1: initial object; else producing task index
    in_fast: bool                   # initial: has a fast copy / produced: output location fast
    in_backing: bool                # a valid backing copy exists at birth
    uses: list[int] = field(default_factory=list)      # task indices that read (or create) it
    mutated_at: set[int] = field(default_factory=set)
    final: str | None = None


def gather_facts(chain: TaskChain) -> dict[str, ObjFacts]:
    facts: dict[str, ObjFacts] = {}
    for o in chain.initial_memory:
        f = facts.get(o.id)
        if f is None:
            f = facts[o.id] = ObjFacts(o.id, o.size, o.type, -1, False, False)
        if o.location == "fast":
            f.in_fast = True
        else:
            f.in_backing = True
    for i, t in enumerate(chain.tasks):
        for out in t.outputs:
            facts[out.id] = ObjFacts(out.id, out.size, out.type, i, out.location == "fast",
                                     out.location == "backing", uses=[i])
        for inp in t.inputs:
            facts[inp].uses.append(i)
        for m in t.mutates_inputs:
            facts[m].mutated_at.add(i)
    for o, loc in chain.final_locations.items():
        if o in facts:
            facts[o].final = loc
    return facts


# --------------------------------------------------------------------------- specs
@dataclass(frozen=True)
class ResidencySpec:
    name: str
    # score(size, distance_tasks, dirty, type) -> larger = evict first
    score: Callable[[int, int, bool, str], float]
    sweep_slack: float = 1.25


def _s_belady(size, dist, dirty, typ):
    return float(dist)


def _s_bytes_dist(size, dist, dirty, typ):
    return float(size) * dist


def _s_largest(size, dist, dirty, typ):
    return float(size) + 1e-6 * dist


def _s_clean_first(size, dist, dirty, typ):
    return (0.0 if dirty else 1e18) + float(size) * dist


_ROLE_W = {"activation": 4.0, "optimizer": 3.0, "gradient": 1.5, "weight": 1.0, "other": 1.0}


def _s_role(size, dist, dirty, typ):
    return _ROLE_W.get(typ, 1.0) * float(size) * dist


RESIDENCY_SPECS: tuple[ResidencySpec, ...] = (
    ResidencySpec("belady", _s_belady),
    ResidencySpec("bytes_x_distance", _s_bytes_dist),
    ResidencySpec("largest", _s_largest, 1.5),
    ResidencySpec("clean_first", _s_clean_first),
    ResidencySpec("role_weighted", _s_role, 2.0),
)


@dataclass(frozen=True)
class PrefetchRule:
    name: str
    kind: str          # "jit" | "window" | "eager"
    param: float = 1.0


PREFETCH_RULES: tuple[PrefetchRule, ...] = (
    PrefetchRule("jit_1.0", "jit", 1.0),
    PrefetchRule("jit_1.25", "jit", 1.25),
    PrefetchRule("jit_1.6", "jit", 1.6),
    PrefetchRule("jit_2.5", "jit", 2.5),
    PrefetchRule("window_1", "window", 1),
    PrefetchRule("window_2", "window", 2),
    PrefetchRule("window_4", "window", 4),
    PrefetchRule("eager", "eager", 0),
)


# --------------------------------------------------------------------------- residency
@dataclass
class Reload:
    obj: str
    need: int           # task index that needs it
    gone_after: int     # task index whose end removes the fast copy (-1: never resident before)
    size: int
    dirty_evict: bool   # the eviction was an offload (reload may have to be deferred behind it)


@dataclass
class Residency:
    releases: dict[int, list[str]]
    offloads: dict[int, list[str]]
    reloads: list[Reload]
    over_budget_tasks: list[int]


def _xfer_us(size: int, bw: int | None) -> float:
    if not bw:
        return 1.0
    return float(max((size + bw - 1) // bw, 1))


def residency_sweep(chain: TaskChain, facts: dict[str, ObjFacts], cap: int | None,
                    spec: ResidencySpec, extra_pressure: dict[int, int] | None = None) -> Residency:
    """``extra_pressure``: bytes to hold free during given tasks on top of what the accounting sees (what a verified run
    reported as in flight there)."""
    tasks = chain.tasks
    extra_pressure = extra_pressure or {}
    n = len(tasks)
    start = [0.0] * (n + 1)
    for i, t in enumerate(tasks):
        start[i + 1] = start[i] + t.runtime
    end = start[1:]
    bw_in = chain.bandwidth_from_slow

    releases: dict[int, list[str]] = {}
    offloads: dict[int, list[str]] = {}
    reloads: list[Reload] = []
    over: list[int] = []
    arrivals: dict[int, list[str]] = {}

    resident: set[str] = set()
    dirty: dict[str, bool] = {}
    use_ptr: dict[str, int] = {o: 0 for o in facts}          # index into uses of the next use
    prev_use: dict[str, int] = {}
    stamp: dict[str, int] = {}
    heap: list[tuple[float, int, str, int]] = []
    charged = 0
    tick = 0

    def window_start(obj: ObjFacts, need: int, lo: int) -> int:
        """First task index during which the reload occupies fast memory."""
        dur = _xfer_us(obj.size, bw_in) * spec.sweep_slack
        anchor = bisect_right(end, start[need] - dur) - 1
        anchor = min(max(anchor, lo), need - 1)
        return anchor + 1

    def push(o: str, now: int) -> None:
        nonlocal tick
        f = facts[o]
        p = use_ptr[o]
        if p >= len(f.uses):
            return
        stamp[o] = stamp.get(o, 0) + 1
        tick += 1
        sc = spec.score(f.size, f.uses[p] - now, dirty.get(o, False), f.type)
        heapq.heappush(heap, (-sc, tick, o, stamp[o]))

    # initial placement
    for f in facts.values():
        if f.birth != -1:
            continue
        if f.in_fast:
            resident.add(f.id)
            dirty[f.id] = not f.in_backing
            charged += f.size
            if f.uses:
                push(f.id, -1)
            elif f.final != "fast":
                releases.setdefault(-1, []).append(f.id)      # never used: handled below
        elif f.uses:
            ws = window_start(f, f.uses[0], -1)
            arrivals.setdefault(ws, []).append(f.id)
            reloads.append(Reload(f.id, f.uses[0], -1, f.size, False))

    # never-used initial fast objects simply stay (nothing can release them before task 0)
    releases.pop(-1, None)

    for i, t in enumerate(tasks):
        for o in arrivals.pop(i, ()):
            if o not in resident:
                resident.add(o)
                dirty[o] = False
                charged += facts[o].size
        touched = set(t.inputs)
        for inp in t.inputs:                      # inputs that arrive exactly now
            if inp not in resident:
                resident.add(inp)
                dirty[inp] = False
                charged += facts[inp].size
        need_now = t.workspace_bytes + extra_pressure.get(i, 0)
        for out in t.outputs:
            if out.location == "fast":
                need_now += out.size
            touched.add(out.id)
        if cap is not None and charged + need_now > cap:
            skipped: list[tuple[float, int, str, int]] = []
            while charged + need_now > cap and heap:
                negsc, tk, o, st = heapq.heappop(heap)
                if stamp.get(o) != st or o not in resident:
                    continue
                f = facts[o]
                p = use_ptr[o]
                if o in touched or p >= len(f.uses) or f.uses[p] <= i:
                    continue                       # an input of this task; re-pushed after it
                nxt = f.uses[p]
                gone = prev_use.get(o, -1)
                ws = window_start(f, nxt, max(gone, -1))
                if ws <= i:
                    continue                       # reload window already open: eviction frees nothing
                if gone < 0 and not f.in_backing:
                    continue                       # initial fast-only object that was never used: cannot move
                if gone < 0:
                    # initial fast copy never used so far: plan it in backing instead
                    f.in_fast = False
                    resident.discard(o)
                    charged -= f.size
                    arrivals.setdefault(ws, []).append(o)
                    reloads.append(Reload(o, nxt, -1, f.size, False))
                    continue
                if dirty.get(o, False):
                    offloads.setdefault(gone, []).append(o)
                else:
                    releases.setdefault(gone, []).append(o)
                resident.discard(o)
                charged -= f.size
                arrivals.setdefault(ws, []).append(o)
                reloads.append(Reload(o, nxt, gone, f.size, dirty.get(o, False)))
            if charged + need_now > cap:
                over.append(i)
        # task runs
        for out in t.outputs:
            if out.location == "fast":
                resident.add(out.id)
                dirty[out.id] = True
                charged += out.size
            use_ptr[out.id] = 1
            prev_use[out.id] = i
            fo = facts[out.id]
            if out.location != "fast" and len(fo.uses) > 1:
                ws = window_start(fo, fo.uses[1], i)
                arrivals.setdefault(ws, []).append(out.id)
                reloads.append(Reload(out.id, fo.uses[1], i, fo.size, False))
        for m in t.mutates_inputs:
            dirty[m] = True
        for inp in t.inputs:
            f = facts[inp]
            p = use_ptr[inp]
            while p < len(f.uses) and f.uses[p] <= i:
                p += 1
            use_ptr[inp] = p
            prev_use[inp] = i
        for o in list(t.inputs) + [x.id for x in t.outputs]:
            if o not in resident:
                continue
            f = facts[o]
            if use_ptr[o] < len(f.uses):
                push(o, i)
                continue
            # last use is behind us
            if f.final == "fast":
                continue
            if f.final == "backing" and (dirty.get(o, False) or not _has_backing(f, offloads, o)):
                offloads.setdefault(i, []).append(o)
            else:
                releases.setdefault(i, []).append(o)
            resident.discard(o)
            charged -= f.size
    return Residency(releases, offloads, reloads, over)


def _has_backing(f: ObjFacts, offloads: dict[int, list[str]], o: str) -> bool:
    if f.in_backing:
        return True
    return any(o in v for v in offloads.values())


# --------------------------------------------------------------------------- prefetch anchors
def assign_anchors(chain: TaskChain, reloads: Sequence[Reload], rule: PrefetchRule) -> dict[str, list[tuple[int, int]]]:
    """obj -> [(anchor_task, need_task)], anchor -1 meaning "preplaced in fast"."""
    tasks = chain.tasks
    n = len(tasks)
    start = [0.0] * (n + 1)
    for i, t in enumerate(tasks):
        start[i + 1] = start[i] + t.runtime
    end = start[1:]
    order = sorted(range(len(reloads)), key=lambda k: (reloads[k].need, k))
    anchors = [0] * len(reloads)
    if rule.kind == "jit":
        limit = float("inf")
        for k in reversed(order):
            r = reloads[k]
            finish = min(start[r.need], limit)
            begin = finish - _xfer_us(r.size, chain.bandwidth_from_slow) * rule.param
            a = bisect_right(end, begin) - 1
            anchors[k] = a
            limit = min(limit, begin)
    elif rule.kind == "window":
        for k in order:
            anchors[k] = reloads[k].need - 1 - int(rule.param)
    else:   # eager: a long fixed look-ahead, bounded below by the eviction point
        for k in order:
            anchors[k] = max(reloads[k].gone_after, reloads[k].need - 9)
    prev = -1
    out: dict[str, list[tuple[int, int]]] = {}
    for k in order:
        r = reloads[k]
        a = min(max(anchors[k], r.gone_after, -1), r.need - 1)
        if rule.kind != "eager":
            a = max(a, prev)                      # FIFO head is always the earliest-needed object
            a = min(a, r.need - 1)
        prev = max(prev, a)
        out.setdefault(r.obj, []).append((a, r.need))
    return out


# --------------------------------------------------------------------------- emit
def emit_plan(chain: TaskChain, facts: dict[str, ObjFacts], res: Residency,
              anchors: dict[str, list[tuple[int, int]]], cap: int | None) -> TaskChain:
    n = len(chain.tasks)
    pre: dict[int, list[tuple[int, str]]] = {}
    preplaced: set[str] = set()
    for obj, lst in anchors.items():
        for a, need in lst:
            if a < 0:
                preplaced.add(obj)
            else:
                pre.setdefault(a, []).append((need, obj))
    new_tasks: list[Task] = []
    for i, t in enumerate(chain.tasks):
        new_tasks.append(replace(
            t,
            releases_after=list(res.releases.get(i, ())),
            offload_after=[TransferTrigger(o) for o in res.offloads.get(i, ())],
            prefetch_after=[TransferTrigger(o) for _, o in sorted(pre.get(i, ()))]))
    initial: list[Object] = []
    seen: set[tuple[str, str]] = set()
    for o in chain.initial_memory:
        f = facts[o.id]
        if o.location == "fast" and not f.in_fast:
            continue                              # the sweep moved this never-used copy to backing
        if (o.id, o.location) not in seen:
            initial.append(o)
            seen.add((o.id, o.location))
    for obj in sorted(preplaced):
        f = facts[obj]
        if (obj, "fast") not in seen:
            initial.append(Object(obj, f.size, "fast", f.type))
            seen.add((obj, "fast"))
    return replace(chain, tasks=new_tasks, initial_memory=initial, fast_memory_capacity=cap)


# --------------------------------------------------------------------------- driver
@dataclass
class Candidate:
    spec: str
    rule: str
    makespan: float | None
    peak_fast: int | None
    error: str | None = None
    repairs: int = 0
    wall_s: float = 0.0

    @property
    def name(self) -> str:
        return f"{self.spec}/{self.rule}"

    @property
    def status(self) -> str:
        return "failed" if self.makespan is None else ("repaired" if self.repairs else "ok")


@dataclass(frozen=True)
class PressureFitDiagnostics:
    """What one planning call did, for logs and for the planner panel: the size of the problem, every candidate with its
    outcome and cost, which one won and by how much."""
    planning_s: float
    task_count: int
    object_count: int
    fast_memory_capacity: int | None
    forced_peak_bytes: int                  # the largest inputs + outputs + workspace of any one task: no plan holds less
    max_task_workspace_bytes: int
    candidate_count: int
    valid_candidate_count: int
    repaired_candidate_count: int
    selected: str
    selected_makespan_us: float
    lower_bound_us: float
    spread: float                           # worst valid makespan / selected makespan
    refined_moves: int
    early_exit: bool
    candidates: tuple[Candidate, ...]

    def format(self, limit: int = 12) -> str:
        cap = "unbounded" if self.fast_memory_capacity is None else f"{self.fast_memory_capacity / 2**30:.2f} GiB"
        lines = [f"PressureFit: {self.task_count} tasks, {self.object_count} objects, fast memory {cap} "
                 f"(largest task holds {self.forced_peak_bytes / 2**30:.2f} GiB), planned in {self.planning_s:.2f} s",
                 f"  {self.valid_candidate_count}/{self.candidate_count} candidates valid ({self.repaired_candidate_count} after repair)"
                 f"{', stopped early at the lower bound' if self.early_exit else ''}; selected {self.selected}: "
                 f"{self.selected_makespan_us:.0f} us = {self.selected_makespan_us / max(self.lower_bound_us, 1e-9):.3f} x lower bound"
                 f"{f', {self.refined_moves} fetches fired earlier' if self.refined_moves else ''}; spread {self.spread:.2f}x"]
        ranked = sorted(self.candidates, key=lambda c: (c.makespan is None, c.makespan or 0.0))
        for c in ranked[:limit]:
            what = f"{c.makespan:.0f} us, peak {c.peak_fast / 2**30:.2f} GiB" if c.makespan is not None else f"failed: {(c.error or '')[:80]}"
            lines.append(f"    {c.name:<28} {c.status:<9} {c.wall_s * 1e3:7.1f} ms  {what}")
        if len(ranked) > limit:
            lines.append(f"    ... {len(ranked) - limit} more")
        return "\n".join(lines)


@dataclass
class PressureFitResult:
    chain: TaskChain
    makespan: float
    peak_fast_bytes: int
    lower_bound: float
    chosen: Candidate
    candidates: list[Candidate]
    early_exit: bool
    planning_s: float = 0.0
    refined_moves: int = 0

    @property
    def idle_fraction(self) -> float:
        return 0.0 if self.makespan <= 0 else 1.0 - self.lower_bound / self.makespan

    def diagnostics(self) -> PressureFitDiagnostics:
        from .spans import static_minimum
        ch = self.chain
        valid = [c for c in self.candidates if c.makespan is not None]
        forced = static_minimum(ch.bare())
        return PressureFitDiagnostics(
            planning_s=self.planning_s, task_count=len(ch.tasks), object_count=len(ch.sizes()),
            fast_memory_capacity=ch.fast_memory_capacity, forced_peak_bytes=int(forced.max(initial=0.0)),
            max_task_workspace_bytes=max((t.workspace_bytes for t in ch.tasks), default=0),
            candidate_count=len(self.candidates), valid_candidate_count=len(valid),
            repaired_candidate_count=sum(1 for c in valid if c.repairs), selected=self.chosen.name,
            selected_makespan_us=self.makespan, lower_bound_us=self.lower_bound,
            spread=max((c.makespan for c in valid), default=self.makespan) / max(self.makespan, 1e-9),
            refined_moves=self.refined_moves, early_exit=self.early_exit, candidates=tuple(self.candidates))


def _build(chain: TaskChain, cap_eff: int | None, cap: int | None, spec: ResidencySpec,
           rule: PrefetchRule, extra_pressure: dict[int, int] | None = None) -> TaskChain:
    facts = gather_facts(chain)
    res = residency_sweep(chain, facts, cap_eff, spec, extra_pressure)
    anchors = assign_anchors(chain, res.reloads, rule)
    return emit_plan(chain, facts, res, anchors, cap)


LOCAL_REPAIRS = 3        # dead-locks answered by holding bytes free at the task that dead-locked (more buys nothing on the corpus and doubles the time)
GLOBAL_REPAIRS = 6       # then by planning against a smaller capacity everywhere


def _verify_candidate(chain: TaskChain, cap: int | None, spec: ResidencySpec, rule: PrefetchRule,
                      max_repairs: int = GLOBAL_REPAIRS, local_repairs: int = LOCAL_REPAIRS):
    """Build, simulate, repair.  The sweep accounts bytes task by task on the stall-free clock; the run can hold more (an
    offload keeps its fast copy until it completes, a fetch that was fired early is charged from its start).  When the run
    dead-locks on fast memory the simulator says at which task and by how many bytes: that much is first held free at
    that task and the two before it (local repair: the rest of the plan is untouched); if the same run keeps failing, the
    whole plan is rebuilt against a smaller capacity (global repair)."""
    cap_eff = cap
    last_err = None
    extra: dict[int, int] = {}
    index = {t.id: i for i, t in enumerate(chain.tasks)}
    local_left = local_repairs if cap is not None else 0
    attempt = 0
    while attempt <= max_repairs + local_repairs:
        planned = _build(chain, cap_eff, cap, spec, rule, extra)
        try:
            log = Simulator(planned).run()
            return planned, log, attempt, None
        except SimulationCapacityError as e:
            last_err = e
            attempt += 1
            if cap is None:
                break
            shrink = int(e.overage_bytes or 0)
            j = index.get(e.task_id or "")
            if local_left > 0 and e.kind == "fast-deadlock" and j is not None and shrink > 0:
                local_left -= 1
                for k in range(max(j - 2, 0), j + 1):
                    extra[k] = extra.get(k, 0) + shrink + (cap >> 7)
                continue
            local_left = 0
            cap_eff = int(min(cap_eff - shrink, cap_eff * 0.94)) if cap_eff else cap_eff
            if cap_eff is None or cap_eff <= 0 or attempt > max_repairs + local_repairs:
                break
        except SimulationError as e:
            last_err = e
            break
    return None, None, attempt, last_err


def pressurefit(chain: TaskChain, fast_memory_capacity: int | None = None, *,
                specs: Sequence[ResidencySpec] | None = None,
                rules: Sequence[PrefetchRule] | None = None,
                early_exit: bool = True, validate: bool = True,
                rel_tolerance: float = 1e-9, refine: bool = True) -> PressureFitResult:
    """Plan ``chain`` under ``fast_memory_capacity`` (defaults to the chain's own field).  ``refine``: fire the fetches the
    winning run waited for earlier where the simulator confirms a gain of more than 0.1 % (``policies.refine``)."""
    import time
    t_begin = time.perf_counter()
    cap = fast_memory_capacity if fast_memory_capacity is not None else chain.fast_memory_capacity
    base = chain.bare()
    if validate:
        validate_planning_input(base)
    lower = compute_lower_bound(base)
    best = None
    cands: list[Candidate] = []
    exited = False
    for spec in (specs or RESIDENCY_SPECS):
        for rule in (rules or PREFETCH_RULES):
            t0 = time.perf_counter()
            planned, log, repairs, err = _verify_candidate(base, cap, spec, rule)
            wall = time.perf_counter() - t0
            if planned is None:
                cands.append(Candidate(spec.name, rule.name, None, None, str(err)[:300], repairs, wall))
                continue
            c = Candidate(spec.name, rule.name, log.makespan, log.peak_fast_memory_bytes, None, repairs, wall)
            cands.append(c)
            if best is None or log.makespan < best[1].makespan - 1e-12:
                best = (planned, log, c)
            if early_exit and log.makespan <= lower * (1 + rel_tolerance) + 1e-9:
                exited = True
                break
        if exited:
            break
    if best is None:
        # last resort: the least residency that can run (every object on the device only while a task touches it, every fetch
        # fired right before its use).  Slow, but when the capacity is a hair above what single tasks need it is the plan that fits
        from .spans import SpanPlan
        t0 = time.perf_counter()
        try:
            planned = SpanPlan(base).fill_min(0.0).emit(cap)
            log = Simulator(planned).run()
            c = Candidate("least_residency", "at_use", log.makespan, log.peak_fast_memory_bytes, None, 0, time.perf_counter() - t0)
            cands.append(c)
            best = (planned, log, c)
        except (SimulationCapacityError, SimulationError) as e:
            cands.append(Candidate("least_residency", "at_use", None, None, str(e)[:300], 0, time.perf_counter() - t0))
    if best is None:
        detail = "; ".join(f"{c.spec}/{c.rule}: {c.error}" for c in cands[:3])
        raise PlanningError(f"no PressureFit candidate fits {cap} bytes of fast memory ({detail})")
    planned, log, c = best
    moves = 0
    if refine and log.stalls:
        from .refine import refine_leads
        p2, l2, moves = refine_leads(planned, log)
        if moves and l2.makespan < log.makespan * 0.999:
            planned, log = p2, l2
        else:
            moves = 0
    return PressureFitResult(planned, log.makespan, log.peak_fast_memory_bytes, lower, c, cands, exited,
                             time.perf_counter() - t_begin, moves)


def apply_pressurefit_policy(chain: TaskChain, fast_memory_capacity: int | None = None, **kw) -> TaskChain:
    return pressurefit(chain, fast_memory_capacity, **kw).chain
