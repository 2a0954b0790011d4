"""Residency plans as spans of tasks, and everything that is common to the planners that work on them.

A ``SpanPlan`` says, for every object, during which tasks it occupies fast memory: a sorted list of disjoint, non-adjacent
spans ``[a, b]`` of task indices (both ends included).  The object is brought in so that it is charged from task ``a`` on (a
prefetch fired after task ``a - 1``, or an initial placement when ``a == 0``) and leaves after task ``b`` (a release when a
current backing copy exists or nothing needs the bytes any more, an offload otherwise).  What has to hold:

    * every task that touches the object (reads it, or produces it in fast memory) lies inside one of its spans;
    * an object produced in fast memory at task ``p`` has a span that starts at ``p``; an initial fast object one that
      starts at 0; an object that must end in fast memory one that ends at the last task.

``level[i]`` is the fast memory charged during task ``i``: the spans that cover ``i`` plus the task's workspace.  Planners
edit spans (``cut``, ``join``, ``move_start``) and the level follows; ``emit`` turns the plan into an annotated chain, and
``verify`` runs it through the simulator, shrinking the capacity the planner works against when bytes in flight (an offload
holds its fast copy until it completes) push the real run over the cap.

The planners built on this: ``max_reduce`` (accounting only), ``min_grow`` (simulator as the oracle), ``roundtrip`` (explicit
lane timelines), ``sliding_window`` (a fixed pattern).
Reference role: the interval plans of ``src/dataflow_sim/policies/{max_reduce,min_grow}.py`` and the shared helpers of
``src/dataflow_sim/policies/_common.py``.
"""
from __future__ import annotations

import bisect
from dataclasses import replace
from typing import Callable

import numpy as np

from ..errors import SimulationCapacityError, SimulationError
from ..schema import Object, TaskChain, TransferTrigger
from ..simulator import Simulator, transfer_runtime
from .pressurefit import ObjFacts, PlanningError, gather_facts


class SpanPlan:
    def __init__(self, chain: TaskChain):
        self.chain = chain
        tasks = chain.tasks
        self.n = n = len(tasks)
        self.facts: dict[str, ObjFacts] = gather_facts(chain)
        self.cum = np.concatenate([[0.0], np.cumsum([t.runtime for t in tasks], dtype=np.float64)])   # stall-free start of task j
        self.workspace = np.array([t.workspace_bytes for t in tasks], dtype=np.float64)
        self.level = self.workspace.copy()
        self.spans: dict[str, list[list[int]]] = {}
        self.touch: dict[str, list[int]] = {}
        self.first_legal: dict[str, int] = {}
        self.tails: list[tuple[str, int, int]] = []          # (object, first task, last task) charged outside spans: offloads in flight
        self.pinned_start: dict[str, bool] = {}
        for o, f in self.facts.items():
            t = sorted(set(f.uses))
            if f.birth >= 0 and not f.in_fast:                 # produced in backing: the producing task does not hold it
                t = [u for u in t if u != f.birth]
            if f.birth < 0 and f.in_fast and (not t or t[0] != 0):
                t = [0] + t                                    # it is there when the chain starts
            if f.final == "fast" and n and (not t or t[-1] != n - 1):
                t = t + [n - 1]
            self.touch[o] = t
            self.first_legal[o] = 0 if f.birth < 0 else (f.birth if f.in_fast else f.birth + 1)
            self.pinned_start[o] = f.in_fast                   # initial fast copy or fast output: the first span cannot start later
            self.spans[o] = []

    # ---------------------------------------------------------------------------------------------------- transfer times
    def tau_in(self, o: str) -> float:
        if not self.chain.bandwidth_from_slow:
            raise PlanningError("the chain gives no bandwidth_from_slow: nothing can be fetched, only plans that keep everything resident exist")
        return transfer_runtime(self.facts[o].size, self.chain.bandwidth_from_slow, None, "from_slow")

    def tau_out(self, o: str) -> float:
        if not self.chain.bandwidth_to_slow:
            raise PlanningError("the chain gives no bandwidth_to_slow: nothing can be offloaded")
        return transfer_runtime(self.facts[o].size, self.chain.bandwidth_to_slow, None, "to_slow")

    def lead_start(self, o: str, need: int, slack: float = 1.0) -> int:
        """The latest task index ``a`` such that a prefetch fired when task ``a`` starts has ``slack`` x its transfer time
        before task ``need`` starts on the stall-free clock (never before the object may exist)."""
        if not self.chain.bandwidth_from_slow:
            return max(self.first_legal[o], 0)
        want = self.cum[need] - self.tau_in(o) * slack
        a = int(np.searchsorted(self.cum, want, side="right")) - 1
        return max(min(a, need), self.first_legal[o], 0)

    def clean_until(self, o: str, b: int) -> bool:
        """True when dropping the object after task ``b`` needs no offload: a backing copy exists from the start and
        nothing has written the object by then (an estimate for scoring; ``emit`` tracks the real state)."""
        f = self.facts[o]
        return f.in_backing and not any(m <= b for m in f.mutated_at)

    def first_free_after(self, o: str, b: int) -> int:
        """The first task during which the object's bytes are free when its span ends at ``b``: the next task, or, when the
        bytes have to be offloaded first, the first one that starts after the offload has had time to complete."""
        if self.clean_until(o, b) or not self.chain.bandwidth_to_slow:
            return b + 1
        done = self.cum[b + 1] + self.tau_out(o)
        return int(np.searchsorted(self.cum, done, side="left"))

    # ----------------------------------------------------------------------------------------------------------- editing
    def _charge(self, o: str, a: int, b: int, sign: float) -> None:
        if b >= a:
            self.level[a:b + 1] += sign * self.facts[o].size

    def add(self, o: str, a: int, b: int) -> None:
        """Add ``[a, b]``, merging with spans it overlaps or touches."""
        spans = self.spans[o]
        keep = []
        for s in spans:
            if s[1] < a - 1 or s[0] > b + 1:
                keep.append(s)
            else:
                self._charge(o, s[0], s[1], -1.0)
                a, b = min(a, s[0]), max(b, s[1])
        self._charge(o, a, b, +1.0)
        keep.append([a, b])
        keep.sort()
        self.spans[o] = keep

    def cut(self, o: str, lo: int, hi: int) -> None:
        """Remove tasks ``lo..hi`` from whichever span holds them (they must hold no touch)."""
        out = []
        for s in self.spans[o]:
            if s[1] < lo or s[0] > hi:
                out.append(s)
                continue
            self._charge(o, max(s[0], lo), min(s[1], hi), -1.0)
            if s[0] < lo:
                out.append([s[0], lo - 1])
            if s[1] > hi:
                out.append([hi + 1, s[1]])
        self.spans[o] = out

    def span_of(self, o: str, i: int) -> int | None:
        for k, s in enumerate(self.spans[o]):
            if s[0] <= i <= s[1]:
                return k
        return None

    def neighbours(self, o: str, i: int) -> tuple[int | None, int | None]:
        """The touches of ``o`` just before and just after task ``i`` (``i`` itself excluded)."""
        t = self.touch[o]
        k = bisect.bisect_left(t, i)
        before = t[k - 1] if k > 0 else None
        k2 = bisect.bisect_right(t, i)
        after = t[k2] if k2 < len(t) else None
        return before, after

    def copy(self) -> "SpanPlan":
        c = object.__new__(SpanPlan)
        c.__dict__.update(self.__dict__)
        c.level = self.level.copy()
        c.spans = {o: [list(s) for s in v] for o, v in self.spans.items()}
        c.tails = list(self.tails)
        return c

    # ------------------------------------------------------------------------------------------------------ seed plans
    def fill_max(self, preplace: Callable[[str], bool] | None = None, slack: float = 1.0) -> "SpanPlan":
        """Everything stays from the earliest point it may exist to its last touch.  Initial backing objects are placed in
        fast memory up front when ``preplace`` says so (default: all), else fetched for their first touch."""
        for o, t in self.touch.items():
            if not t:
                continue
            f = self.facts[o]
            a = self.first_legal[o]
            if f.birth < 0 and not f.in_fast and preplace is not None and not preplace(o):
                a = self.lead_start(o, t[0], slack)
            self.add(o, min(a, t[0]), t[-1])
        return self

    def fill_min(self, slack: float = 1.0) -> "SpanPlan":
        """Every touch gets its own span, opened just early enough for the fetch."""
        for o, t in self.touch.items():
            for j, u in enumerate(t):
                if j == 0 and self.pinned_start[o]:
                    self.add(o, u, u)
                else:
                    self.add(o, self.lead_start(o, u, slack), u)
        return self

    def check(self) -> None:
        for o, t in self.touch.items():
            for u in t:
                if self.span_of(o, u) is None:
                    raise AssertionError(f"{o!r} is touched by task {u} outside its spans {self.spans[o]}")
            if t and self.pinned_start[o] and self.spans[o][0][0] != t[0]:
                raise AssertionError(f"{o!r} exists in fast memory from task {t[0]}, its first span starts at {self.spans[o][0][0]}")

    # ---------------------------------------------------------------------------------------------------------- emission
    def emit(self, cap: int | None) -> TaskChain:
        chain, n = self.chain, self.n
        rel: dict[int, list[str]] = {}
        off: dict[int, list[str]] = {}
        pre: dict[int, list[tuple[int, str]]] = {}
        preplaced: list[str] = []
        for o, spans in self.spans.items():
            f = self.facts[o]
            backing_valid = f.in_backing
            muts = sorted(f.mutated_at)
            for k, (a, b) in enumerate(spans):
                born_here = f.birth == a and f.in_fast
                if born_here:
                    backing_valid = False
                elif not (f.birth < 0 and f.in_fast and k == 0):
                    if a == 0 and f.birth < 0:
                        preplaced.append(o)
                    else:
                        need = next((u for u in self.touch[o] if u >= a), b)
                        pre.setdefault(a - 1, []).append((need, o))
                j = bisect.bisect_left(muts, a)
                if j < len(muts) and muts[j] <= b:
                    backing_valid = False
                last = k == len(spans) - 1
                if last and f.final == "fast":
                    continue
                if (not last or f.final == "backing") and not backing_valid:
                    off.setdefault(b, []).append(o)
                    backing_valid = True
                else:
                    rel.setdefault(b, []).append(o)
        tasks = [replace(t, releases_after=sorted(rel.get(i, ())),
                         offload_after=[TransferTrigger(o) for o in sorted(off.get(i, ()))],
                         prefetch_after=[TransferTrigger(o) for _, o in sorted(pre.get(i, ()))])
                 for i, t in enumerate(chain.tasks)]
        initial = list(chain.initial_memory)
        have = {(x.id, x.location) for x in initial}
        for o in sorted(preplaced):
            if (o, "fast") not in have:
                initial.append(Object(o, self.facts[o].size, "fast", self.facts[o].type))
        return replace(chain, tasks=tasks, initial_memory=initial, fast_memory_capacity=cap)


def check_input(chain: TaskChain, cap: int | None, name: str) -> None:
    """Refuse a malformed chain (``ValidationError``) and say ``PlanningError`` when the chain is fine but some task's own
    operands exceed the capacity: that is an answer about the capacity, which callers that search over budgets expect."""
    from ..validate import ValidationError, validate_planning_input
    try:
        validate_planning_input(replace(chain, fast_memory_capacity=cap))
    except ValidationError as e:
        if set(e.rules) <= {"task-cannot-fit", "initial-overflow"}:
            raise PlanningError(f"{name}: {e.problems[0]}") from None
        raise


def static_minimum(chain: TaskChain) -> np.ndarray:
    """Bytes no plan can avoid holding during each task: its inputs, its fast outputs and its workspace."""
    sizes = chain.sizes()
    return np.array([sum(sizes[i] for i in set(t.inputs)) + sum(o.size for o in t.outputs if o.location == "fast") + t.workspace_bytes
                     for t in chain.tasks], dtype=np.float64)


def verify(build: Callable[[int | None], TaskChain], cap: int | None, name: str, max_repairs: int = 8):
    """Simulate what ``build(cap_eff)`` returns; when the run dead-locks on fast memory (bytes in flight the accounting did
    not see) rebuild against a smaller effective capacity.  Returns ``(planned, log, repairs)``."""
    cap_eff = cap
    err: Exception | None = None
    for attempt in range(max_repairs + 1):
        try:
            planned = build(cap_eff)
        except PlanningError as e:
            err = err or e
            break
        try:
            return planned, Simulator(planned).run(), attempt
        except SimulationCapacityError as e:
            err = e
            if cap is None or e.kind != "fast-deadlock":
                break
            cap_eff = int(min(cap_eff - int(e.overage_bytes or 0), cap_eff * 0.95))
            if cap_eff <= 0:
                break
        except SimulationError as e:
            err = e
            break
    raise PlanningError(f"{name}: {err}") from None


class LaneTimeline:
    """Booked intervals on one copy lane (one transfer at a time)."""

    def __init__(self):
        self.starts: list[float] = []
        self.ends: list[float] = []

    def earliest(self, t0: float, length: float) -> float:
        """The earliest start at or after ``t0`` of a free interval of ``length``."""
        k = bisect.bisect_right(self.ends, t0)
        t = t0
        while k < len(self.starts):
            if self.starts[k] - t >= length:
                return t
            t = max(t, self.ends[k])
            k += 1
        return t

    def latest(self, t1: float, length: float, not_before: float = 0.0) -> float | None:
        """The latest start of a free interval of ``length`` that ends at or before ``t1`` and starts at or after
        ``not_before``; None when there is none."""
        k = bisect.bisect_left(self.starts, t1) - 1
        end = t1
        while True:
            lo = self.ends[k] if k >= 0 else 0.0
            if k >= 0 and self.ends[k] > end:                      # this booking overlaps the window's end
                end = min(end, self.starts[k])
                k -= 1
                continue
            if end - max(lo, not_before) >= length:
                return end - length
            if k < 0 or end - length < not_before:
                return None
            end = min(end, self.starts[k])
            k -= 1

    def book(self, start: float, length: float) -> None:
        k = bisect.bisect_left(self.starts, start)
        self.starts.insert(k, start)
        self.ends.insert(k, start + length)
