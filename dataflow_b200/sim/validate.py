"""Static validation of TaskChains: everything that can be decided without advancing the simulator's clock.

The validator runs in four stages, each a function from a chain to a list of ``Problem`` records; a later stage runs only
when the earlier ones found nothing, because it takes their guarantees for granted:

    ids          every id a task names exists by then; ids are fresh and unrepeated; ``mutates_inputs`` names inputs of the
                 same task and ``releases_after`` objects that exist; locations and sizes are sane;
                 transfers without a runtime have a bandwidth to be priced with
    transfers    a walk over the chain that tracks where each object's copies are: a prefetch needs a backing copy and no fast
                 copy, an offload needs a fast copy, no object is moved twice in one direction by one task (both ways is
                 allowed: the fetch waits for the offload, which is how a plan parks bytes across one long task)
    lifetimes    the same walk with dirty bits: a task's inputs are resident when it starts, a release does not throw away the
                 only valid copy of bytes something later reads, ``final_locations`` are met with current bytes
    capacity     the initial objects fit their memories, and every task's inputs + fast outputs + workspace fit fast memory
                 (no plan can run a task whose own footprint does not fit)

Unlike the simulator, which stops at the first violation it runs into, every stage reports ALL of its problems, each with
a rule code that tests and tools match on (``Problem.rule``), the task and the object.  Timing properties (lane contention,
stalls, bytes in flight) are not static and are left to the simulator.

``validate_chain`` runs all stages on an annotated chain; ``validate_planning_input`` runs ``ids`` and ``capacity`` on a
chain a planner is about to annotate and refuses one that already carries a plan.
Reference role: ``src/dataflow_sim/core/validate.py:52-455``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Iterable

from .schema import TaskChain

RULES = {
    # ids
    "bad-location": "a location other than fast / backing",
    "negative-size": "an object, output or workspace of negative size; a negative runtime or capacity",
    "duplicate-initial-object": "an initial object listed twice at one location, or with two sizes",
    "duplicate-task-id": "two tasks with one id",
    "duplicate-input": "an input listed twice by one task",
    "unknown-input": "an input no initial object or earlier output provides",
    "output-reuses-id": "an output whose id already exists",
    "mutation-not-an-input": "mutates_inputs names something the task does not read",
    "unknown-release-object": "releases_after names an id that does not exist by then",
    "unknown-transfer-object": "a prefetch or offload of an id that does not exist by then",
    "unknown-final-object": "final_locations names an id the chain never creates",
    "missing-bandwidth": "a transfer without a runtime on a chain without that direction's bandwidth",
    # transfers
    "prefetch-already-resident": "a prefetch of an object that has a fast copy",
    "prefetch-without-backing-copy": "a prefetch of an object that has no backing copy",
    "offload-not-resident": "an offload of an object that has no fast copy",
    "duplicate-transfer": "one task moves one object twice in one direction",
    "release-and-offload": "one task both releases and offloads one object",
    "release-not-resident": "a release of an object that has no fast copy",
    "duplicate-release": "one task releases one object twice",
    # lifetimes
    "input-not-resident": "a task reads an object whose fast copy is gone and was not brought back",
    "prefetch-never-used": "a prefetch of an object that nothing reads afterwards and that need not end in fast memory",
    "release-loses-data": "a release drops the only current copy of bytes that are read, fetched or required later",
    "final-not-on-backing": "final_locations wants a backing copy that does not exist",
    "final-backing-stale": "final_locations wants a backing copy, and the one there is older than the fast copy",
    "final-not-on-fast": "final_locations wants a fast copy that does not exist",
    # capacity
    "initial-overflow": "the initial objects exceed a memory's capacity",
    "task-cannot-fit": "a task's inputs, fast outputs and workspace exceed fast memory",
    # planning input
    "already-planned": "a planner's input that carries releases or transfers",
}


@dataclass(frozen=True)
class Problem:
    rule: str
    detail: str
    task: str | None = None
    obj: str | None = None

    def __str__(self) -> str:
        where = f"task {self.task!r}: " if self.task is not None else ""
        return f"{self.rule}: {where}{self.detail}"


class ValidationError(ValueError):
    """Raised with every problem the failing stage found.  ``problems``: their texts, ``found``: the records,
    ``rules``: the distinct rule codes in the order met."""

    def __init__(self, problems: Iterable):
        self.found = [p if isinstance(p, Problem) else Problem("invalid", str(p)) for p in problems]
        self.problems = [str(p) for p in self.found]
        self.rules = list(dict.fromkeys(p.rule for p in self.found))
        super().__init__("invalid chain:\n  - " + "\n  - ".join(self.problems))


# --------------------------------------------------------------------------------------------------------------- stage: ids
def check_ids(chain: TaskChain) -> list[Problem]:
    out: list[Problem] = []
    add = lambda rule, detail, task=None, obj=None: out.append(Problem(rule, detail, task, obj))
    sizes: dict[str, int] = {}
    seen: set[tuple[str, str]] = set()
    for o in chain.initial_memory:
        if o.location not in ("fast", "backing"):
            add("bad-location", f"initial object {o.id!r} is at {o.location!r}", obj=o.id)
        if (o.id, o.location) in seen:
            add("duplicate-initial-object", f"{o.id!r} is listed twice at {o.location!r}", obj=o.id)
        seen.add((o.id, o.location))
        if o.size < 0:
            add("negative-size", f"initial object {o.id!r} has size {o.size}", obj=o.id)
        if o.id in sizes and sizes[o.id] != o.size:
            add("duplicate-initial-object", f"the copies of {o.id!r} have sizes {sizes[o.id]} and {o.size}", obj=o.id)
        sizes[o.id] = o.size
    ids: set[str] = set()
    need = {"from_slow": False, "to_slow": False}
    for t in chain.tasks:
        if t.id in ids:
            add("duplicate-task-id", "the id is used by an earlier task", t.id)
        ids.add(t.id)
        if t.runtime < 0:
            add("negative-size", f"runtime {t.runtime}", t.id)
        if t.workspace_bytes < 0:
            add("negative-size", f"workspace of {t.workspace_bytes} bytes", t.id)
        once: set[str] = set()
        for i in t.inputs:
            if i in once:
                add("duplicate-input", f"reads {i!r} twice", t.id, i)
            once.add(i)
            if i not in sizes:
                add("unknown-input", f"reads {i!r}, which nothing has provided by then", t.id, i)
        for m in t.mutates_inputs:
            if m not in once:
                add("mutation-not-an-input", f"mutates {m!r} without reading it", t.id, m)
        for o in t.outputs:
            if o.id in sizes:
                add("output-reuses-id", f"output {o.id!r} already exists", t.id, o.id)
            if o.size < 0:
                add("negative-size", f"output {o.id!r} has size {o.size}", t.id, o.id)
            if o.location not in ("fast", "backing"):
                add("bad-location", f"output {o.id!r} goes to {o.location!r}", t.id, o.id)
            sizes[o.id] = o.size
        for r in t.releases_after:                        # any object may be dropped after any task, not only the task's own
            if r not in sizes:
                add("unknown-release-object", f"releases {r!r}, which does not exist by then", t.id, r)
        for direction, trigs in (("to_slow", t.offload_after), ("from_slow", t.prefetch_after)):
            for tr in trigs:
                if tr.obj_id not in sizes:
                    verb = "offloads" if direction == "to_slow" else "prefetches"
                    add("unknown-transfer-object", f"{verb} {tr.obj_id!r}, which does not exist by then", t.id, tr.obj_id)
                if tr.runtime is None:
                    need[direction] = True
                elif tr.runtime < 0:
                    add("negative-size", f"transfer of {tr.obj_id!r} with runtime {tr.runtime}", t.id, tr.obj_id)
    if need["from_slow"] and not chain.bandwidth_from_slow:
        add("missing-bandwidth", "prefetches without a runtime need bandwidth_from_slow")
    if need["to_slow"] and not chain.bandwidth_to_slow:
        add("missing-bandwidth", "offloads without a runtime need bandwidth_to_slow")
    for o, loc in chain.final_locations.items():
        if o not in sizes:
            add("unknown-final-object", f"final_locations names {o!r}", obj=o)
        if loc not in ("fast", "backing"):
            add("bad-location", f"final_locations[{o!r}] is {loc!r}", obj=o)
    for cap in ("fast_memory_capacity", "backing_memory_capacity"):
        v = getattr(chain, cap)
        if v is not None and v < 0:
            add("negative-size", f"{cap} is {v}")
    return out


# ------------------------------------------------------------------------------------------- the residency walk (two stages)
class _Residency:
    """Where each object's copies are after each task, timing ignored: an offload has dropped the fast copy, a prefetch has
    restored it, by the next task; a task that releases and prefetches one object drops the copy and queues a fresh fetch.
    ``dirty``: the fast copy is newer than the backing copy (or there is none)."""

    def __init__(self, chain: TaskChain):
        self.fast: set[str] = set()
        self.backing: set[str] = set()
        self.dirty: set[str] = set()
        for o in chain.initial_memory:
            (self.fast if o.location == "fast" else self.backing).add(o.id)
        for o in chain.initial_memory:
            if o.location == "fast" and o.id not in self.backing:
                self.dirty.add(o.id)                      # the only copy: losing it loses the bytes

    def commit(self, t) -> None:
        for o in t.outputs:
            if o.location == "fast":
                self.fast.add(o.id)
                self.dirty.add(o.id)
            else:
                self.backing.add(o.id)
        self.dirty.update(t.mutates_inputs)
        for tr in t.offload_after:
            self.backing.add(tr.obj_id)
            self.dirty.discard(tr.obj_id)
            self.fast.discard(tr.obj_id)
        for r in t.releases_after:                        # a release frees at once; a prefetch of the same task queues after it
            self.fast.discard(r)
            self.dirty.discard(r)
        for tr in t.prefetch_after:
            self.fast.add(tr.obj_id)


def check_transfers(chain: TaskChain) -> list[Problem]:
    out: list[Problem] = []
    st = _Residency(chain)
    for t in chain.tasks:
        off = [x.obj_id for x in t.offload_after]
        pre = [x.obj_id for x in t.prefetch_after]
        for name, ids in (("offloads", off), ("prefetches", pre)):
            for o in sorted({x for x in ids if ids.count(x) > 1}):
                out.append(Problem("duplicate-transfer", f"{name} {o!r} {ids.count(o)} times", t.id, o))
        for o in sorted(set(off) & set(t.releases_after)):
            out.append(Problem("release-and-offload", f"releases and offloads {o!r}: the offload already frees the fast copy", t.id, o))
        produced_fast = {o.id for o in t.outputs if o.location == "fast"}
        produced_backing = {o.id for o in t.outputs if o.location == "backing"}
        for o in dict.fromkeys(off):
            if o not in st.fast and o not in produced_fast:
                out.append(Problem("offload-not-resident", f"offloads {o!r}, which has no fast copy", t.id, o))
        for o in sorted({x for x in t.releases_after if t.releases_after.count(x) > 1}):
            out.append(Problem("duplicate-release", f"releases {o!r} {t.releases_after.count(o)} times", t.id, o))
        for o in dict.fromkeys(t.releases_after):
            if o not in st.fast and o not in produced_fast:
                out.append(Problem("release-not-resident", f"releases {o!r}, which has no fast copy", t.id, o))
        for o in dict.fromkeys(pre):
            if o in set(off):
                continue                                   # the fetch waits for this task's offload, which makes the backing copy
            if (o in st.fast or o in produced_fast) and o not in t.releases_after:
                out.append(Problem("prefetch-already-resident", f"prefetches {o!r}, which is in fast memory", t.id, o))
            elif o not in st.backing and o not in produced_backing:
                # (also when this task drops the fast copy first: dropping it does not make a backing copy)
                out.append(Problem("prefetch-without-backing-copy", f"prefetches {o!r}, which has no backing copy", t.id, o))
        st.commit(t)
    return out


def check_lifetimes(chain: TaskChain) -> list[Problem]:
    out: list[Problem] = []
    st = _Residency(chain)
    # where each object is referenced next: as an input, by a prefetch, or by a final location that needs its bytes
    later_use: dict[str, list[int]] = {}
    for i, t in enumerate(chain.tasks):
        for o in list(t.inputs) + [x.obj_id for x in t.prefetch_after]:
            later_use.setdefault(o, []).append(i)
    n = len(chain.tasks)
    for o in chain.final_locations:
        later_use.setdefault(o, []).append(n)
    reads: dict[str, list[int]] = {}
    for i, t in enumerate(chain.tasks):
        for o in t.inputs:
            reads.setdefault(o, []).append(i)
    for i, t in enumerate(chain.tasks):
        for o in t.inputs:
            if o not in st.fast:
                how = "only a backing copy exists" if o in st.backing else "no copy exists"
                out.append(Problem("input-not-resident", f"reads {o!r}, but {how} and nothing brought it back", t.id, o))
        for tr in t.prefetch_after:
            o = tr.obj_id
            if not any(j > i for j in reads.get(o, ())) and chain.final_locations.get(o) != "fast":
                # (the simulator frees every copy of an object at a release past its last reference, so such a fetch can
                # also find its source gone)
                out.append(Problem("prefetch-never-used", f"prefetches {o!r}, which no later task reads", t.id, o))
        dirty_after = (st.dirty | set(t.mutates_inputs) | {o.id for o in t.outputs if o.location == "fast"})
        for r in t.releases_after:
            if r in {x.obj_id for x in t.offload_after}:
                continue                                   # reported by the transfers stage
            used_later = any(j > i for j in later_use.get(r, ()))
            if used_later and (r in dirty_after or r not in st.backing):
                why = "the backing copy is older than the bytes released" if r in st.backing else "there is no backing copy"
                out.append(Problem("release-loses-data", f"releases {r!r}, which is used later, and {why}", t.id, r))
        st.commit(t)
    for o, loc in chain.final_locations.items():
        if loc == "backing":
            if o not in st.backing:
                out.append(Problem("final-not-on-backing", f"{o!r} has no backing copy at the end", obj=o))
            elif o in st.dirty:
                out.append(Problem("final-backing-stale", f"the fast copy of {o!r} was changed after its last offload", obj=o))
        elif loc == "fast" and o not in st.fast:
            out.append(Problem("final-not-on-fast", f"{o!r} is not in fast memory at the end", obj=o))
    return out


# ---------------------------------------------------------------------------------------------------------- stage: capacity
def check_capacity(chain: TaskChain) -> list[Problem]:
    out: list[Problem] = []
    held = {"fast": 0, "backing": 0}
    for o in chain.initial_memory:
        held[o.location] = held.get(o.location, 0) + o.size
    for loc, cap in (("fast", chain.fast_memory_capacity), ("backing", chain.backing_memory_capacity)):
        if cap is not None and held[loc] > cap:
            out.append(Problem("initial-overflow", f"the initial objects take {held[loc]} bytes of {loc} memory, capacity {cap}"))
    cap = chain.fast_memory_capacity
    if cap is None:
        return out
    sizes = {o.id: o.size for o in chain.initial_memory}
    for t in chain.tasks:
        ins = sum(sizes.get(i, 0) for i in set(t.inputs))
        outs = sum(o.size for o in t.outputs if o.location == "fast")
        if ins + outs + t.workspace_bytes > cap:
            out.append(Problem("task-cannot-fit", f"{ins} bytes of inputs + {outs} of fast outputs + {t.workspace_bytes} of workspace "
                                                  f"= {ins + outs + t.workspace_bytes} > fast capacity {cap}", t.id))
        for o in t.outputs:
            sizes[o.id] = o.size
    return out


STAGES: dict[str, Callable[[TaskChain], list[Problem]]] = {
    "ids": check_ids, "transfers": check_transfers, "lifetimes": check_lifetimes, "capacity": check_capacity}


def chain_problems(chain: TaskChain, stages: Iterable[str] = ("ids", "transfers", "lifetimes", "capacity")) -> list[Problem]:
    """The problems of the first stage that finds any (later stages assume the earlier ones passed)."""
    for s in stages:
        found = STAGES[s](chain)
        if found:
            return found
    return []


def validate_chain(chain: TaskChain) -> TaskChain:
    probs = chain_problems(chain)
    if probs:
        raise ValidationError(probs)
    return chain


def validate_planning_input(chain: TaskChain) -> TaskChain:
    probs = chain_problems(chain, ("ids", "capacity"))
    if not probs:
        for t in chain.tasks:
            if t.releases_after or t.offload_after or t.prefetch_after:
                probs = [Problem("already-planned", "carries releases or transfers; planners take a bare chain", t.id)]
                break
    if probs:
        raise ValidationError(probs)
    return chain
