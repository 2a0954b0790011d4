"""Event-driven simulator of an annotated TaskChain.

Three lanes: one compute lane (tasks in chain order, one at a time), one
``from_slow`` (backing → fast) FIFO and one ``to_slow`` (fast → backing) FIFO,
each with at most one transfer in flight.  The rules are the ones the executor
implements, so that the executor on a virtual-time backend reproduces this log
exactly:

* A task starts at the earliest time the compute lane is free, every input is
  ``live`` in fast memory and the fast ledger admits its fast outputs plus its
  opaque workspace.  Outputs are charged at task start.
* A transfer is charged at its destination when it *starts*, never when it is
  queued; a head that does not fit blocks its lane until bytes free up.
* An offload frees the fast copy when it completes; a release frees it at once.
  A release past the object's last reference, with no ``final_locations`` entry,
  frees the backing copy too ("dead everywhere").
* A prefetch fired while the same object's offload is queued or in flight is
  deferred and joins the ``from_slow`` queue when that offload completes.
* Event order at equal times: ``from_slow`` completion, ``to_slow`` completion,
  task completion.  After every event both lane heads are retried, ``from_slow``
  first.
* Transfer time is ``max(ceil(size / bandwidth), 1)`` unless the trigger carries
  an explicit runtime.

Behavioural parity: reference ``src/dataflow_sim/engine/simulator.py:141-889``
(lanes, deferred prefetch, dead-everywhere, workspace charge, tie order).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable

from .errors import SimulationCapacityError, SimulationError
from .schema import Event, EventLog, MemoryTracePoint, Task, TaskChain, TaskInterval

INF = float("inf")
FAST = "fast"
BACKING = "backing"


class _Entry:
    __slots__ = ("size", "state", "type", "dirty")

    def __init__(self, size: int, state: str, type_: str = "other", dirty: bool = False):
        self.size = size
        self.state = state
        self.type = type_
        self.dirty = dirty        # fast copy newer than (or without) a backing copy


@dataclass
class _Xfer:
    obj: str
    direction: str
    size: int
    runtime: float
    type: str = "other"
    start: float = 0.0
    end: float = 0.0


def transfer_runtime(size: int, bandwidth: int | None, override: float | None, direction: str = "?") -> float:
    if override is not None:
        return max(float(override), 0.0)
    if not bandwidth:
        raise SimulationError(f"{direction} transfer needs a bandwidth on the chain or a per-trigger runtime")
    return float(max((size + bandwidth - 1) // bandwidth, 1))


def last_references(tasks: Iterable[Task]) -> dict[str, int]:
    last: dict[str, int] = {}
    for i, t in enumerate(tasks):
        for o in t.inputs:
            last[o] = i
        for tr in t.offload_after:
            last[tr.obj_id] = i
        for tr in t.prefetch_after:
            last[tr.obj_id] = i
    return last


class Simulator:
    """One run over one chain.  Use :func:`run` unless you need the internals."""

    def __init__(self, chain: TaskChain, *, events: bool = False, memory_trace: bool = False,
                 check_dirty_release: bool = True):
        self.chain = chain
        self.want_events = events
        self.want_trace = memory_trace
        self.check_dirty_release = check_dirty_release
        self.pool: dict[tuple[str, str], _Entry] = {}
        self.used = {FAST: 0, BACKING: 0}
        self.cap = {FAST: chain.fast_memory_capacity, BACKING: chain.backing_memory_capacity}
        self.workspace = 0
        self.queue: dict[str, list[_Xfer]] = {"from_slow": [], "to_slow": []}
        self.flight: dict[str, _Xfer | None] = {"from_slow": None, "to_slow": None}
        self.deferred: dict[str, list[_Xfer]] = {}
        self.seq: dict[tuple[str, str], int] = {}
        self.intervals: list[TaskInterval] = []
        self.events: list[Event] = []
        self.trace: list[MemoryTracePoint] = []
        self.peak_fast = 0
        self.peak_backing = 0
        self.stalls: dict[str, float] = {}
        self.stall_causes: dict[str, tuple[tuple[str, ...], bool]] = {}
        self.last_ref = last_references(chain.tasks)

    # -- bookkeeping ---------------------------------------------------------
    def _note(self, kind: str, t: float, **kw) -> None:
        f = self.used[FAST] + self.workspace
        if f > self.peak_fast:
            self.peak_fast = f
        if self.used[BACKING] > self.peak_backing:
            self.peak_backing = self.used[BACKING]
        if self.want_trace:
            if not self.trace or self.trace[-1].t != t or self.trace[-1].fast_bytes != self.used[FAST]:
                self.trace.append(MemoryTracePoint(t, self.used[FAST], self.workspace))
        if self.want_events:
            self.events.append(Event(t=t, kind=kind, fast_bytes=self.used[FAST],
                                     backing_bytes=self.used[BACKING], **kw))

    def _free(self, loc: str) -> float:
        cap = self.cap[loc]
        if cap is None:
            return INF
        return cap - self.used[loc] - (self.workspace if loc == FAST else 0)

    # -- lanes ----------------------------------------------------------------
    def _try_start(self, direction: str, now: float) -> bool:
        if self.flight[direction] is not None or not self.queue[direction]:
            return False
        tx = self.queue[direction][0]
        dst = FAST if direction == "from_slow" else BACKING
        existing = self.pool.get((tx.obj, dst))
        if self._free(dst) + (existing.size if existing is not None else 0) < tx.size:
            return False
        self.queue[direction].pop(0)
        if direction == "from_slow":
            if existing is None:
                self.pool[(tx.obj, FAST)] = _Entry(tx.size, "inbound", tx.type)
                self.used[FAST] += tx.size
            else:
                existing.state = "inbound"
        else:
            self.pool[(tx.obj, FAST)].state = "outbound"
            if existing is None:
                self.pool[(tx.obj, BACKING)] = _Entry(tx.size, "inbound", tx.type)
                self.used[BACKING] += tx.size
            else:
                if existing.size != tx.size:
                    raise SimulationError(f"to_slow overwrite size mismatch for {tx.obj!r}")
                existing.state = "inbound"
        tx.start, tx.end = now, now + tx.runtime
        self.flight[direction] = tx
        n = self.seq.get((direction, tx.obj), 0)
        self.seq[(direction, tx.obj)] = n + 1
        name = f"{direction}:{tx.obj}" if n == 0 else f"{direction}:{tx.obj}#{n}"
        self.intervals.append(TaskInterval(name, tx.start, tx.end, direction))
        self._note("transfer_start", now, transfer_obj=tx.obj, transfer_direction=direction)
        return True

    def _poke(self, now: float) -> None:
        # a start on one lane can never unblock the other (it only charges bytes)
        self._try_start("from_slow", now)
        self._try_start("to_slow", now)

    def _complete(self, direction: str) -> float:
        tx = self.flight[direction]
        assert tx is not None
        t = tx.end
        if direction == "from_slow":
            e = self.pool[(tx.obj, FAST)]
            e.state, e.dirty = "live", False
        else:
            src = self.pool.pop((tx.obj, FAST))
            self.used[FAST] -= src.size
            self.pool[(tx.obj, BACKING)].state = "live"
        self.flight[direction] = None
        self._note("transfer_end", t, transfer_obj=tx.obj, transfer_direction=direction)
        if direction == "to_slow":
            for w in self.deferred.pop(tx.obj, ()):
                self.queue["from_slow"].append(w)
                self._note("transfer_enqueue", t, transfer_obj=w.obj, transfer_direction="from_slow")
        self._poke(t)
        return t

    def _next_completion(self) -> tuple[float, str | None]:
        a, b = self.flight["from_slow"], self.flight["to_slow"]
        ta = a.end if a is not None else INF
        tb = b.end if b is not None else INF
        if ta == INF and tb == INF:
            return INF, None
        return (ta, "from_slow") if ta <= tb else (tb, "to_slow")

    def _advance(self, until: float) -> None:
        """Retire every transfer that ends at or before ``until`` in event order."""
        while True:
            t, d = self._next_completion()
            if d is None or t > until:
                return
            self._complete(d)

    # -- tasks ----------------------------------------------------------------
    def _before_directives(self, idx: int, task: Task, t: float) -> None:
        """Hook for planners that decide a task's directives while the run unfolds (``policies.lookahead``)."""

    def _on_deadlock(self, idx: int, task: Task, now: float, need: int, missing: list[str]) -> bool:
        """Hook: return True after making progress possible (planners add an emergency eviction)."""
        return False

    def _blocked_reason(self, task: Task, need: int):
        missing = [i for i in task.inputs
                   if (e := self.pool.get((i, FAST))) is None or e.state != "live"]
        short = self.cap[FAST] is not None and self.used[FAST] + need > self.cap[FAST]
        return missing, short

    def _deadlock(self, task: Task, now: float, need: int, missing: list[str]):
        cap = self.cap[FAST]
        actual = over = None
        parts = []
        if missing:
            parts.append(f"inputs {missing} not live in fast memory")
        if cap is not None and self.used[FAST] + need > cap:
            actual = self.used[FAST] + need
            over = actual - cap
            parts.append(f"fast memory {self.used[FAST]} + {need} needed > cap {cap} with nothing in flight")
        resident = tuple(sorted(((k[0], e.size) for k, e in self.pool.items() if k[1] == FAST),
                                key=lambda x: -x[1]))[:32]
        raise SimulationCapacityError(
            f"task {task.id!r} deadlocked at t={now}: " + "; ".join(parts),
            kind="fast-deadlock", task_id=task.id, capacity_bytes=cap, actual_need_bytes=actual,
            overage_bytes=over, missing_object_ids=tuple(missing), time=now, resident=resident)

    def _settle_task(self, idx: int, task: Task, t: float) -> None:
        """The task has ended: its workspace is gone, its outputs are live, what it wrote is dirty."""
        pool = self.pool
        self.workspace = 0
        for out in task.outputs:
            e = pool[(out.id, out.location)]
            e.state = "live"
            e.dirty = out.location == FAST
        for m in task.mutates_inputs:
            pool[(m, FAST)].dirty = True
        self._note("task_end", t, task_id=task.id)

    def _finish_task(self, idx: int, task: Task, t: float) -> None:
        self._settle_task(idx, task, t)
        self._before_directives(idx, task, t)
        self._apply_directives(idx, task, t)

    def _apply_directives(self, idx: int, task: Task, t: float) -> None:
        """Releases first (they free at once), then offloads and prefetches join their lanes, then both lanes are retried."""
        pool, used = self.pool, self.used
        if task.releases_after:
            for obj in task.releases_after:
                e = pool.get((obj, FAST))
                if e is None:
                    raise SimulationError(f"task {task.id!r} cannot release {obj!r}: no fast copy")
                if e.state != "live":
                    raise SimulationError(f"task {task.id!r} cannot release {obj!r}: state={e.state!r}")
                dead = idx >= self.last_ref.get(obj, -1) and obj not in self.chain.final_locations
                if self.check_dirty_release and e.dirty and not dead:
                    raise SimulationError(
                        f"task {task.id!r} releases {obj!r} whose fast copy is the only current version "
                        f"and it is still needed — offload it instead")
                used[FAST] -= e.size
                del pool[(obj, FAST)]
                if dead:
                    b = pool.get((obj, BACKING))
                    if b is not None and b.state == "live":
                        used[BACKING] -= b.size
                        del pool[(obj, BACKING)]
            self._note("release", t, object_ids=tuple(task.releases_after))
        ch = self.chain
        for trig in task.offload_after:
            src = pool.get((trig.obj_id, FAST))
            if src is None or src.state != "live":
                raise SimulationError(f"task {task.id!r} cannot offload {trig.obj_id!r}: fast state="
                                      f"{src.state if src else 'absent'!r}")
            b = pool.get((trig.obj_id, BACKING))
            if b is not None and (b.state != "live" or b.size != src.size):
                raise SimulationError(f"task {task.id!r} cannot offload {trig.obj_id!r}: backing entry "
                                      f"state={b.state!r} size={b.size}")
            src.state = "pending_outbound"
            self.queue["to_slow"].append(_Xfer(trig.obj_id, "to_slow", src.size,
                                               transfer_runtime(src.size, ch.bandwidth_to_slow, trig.runtime, "to_slow"),
                                               src.type))
            self._note("transfer_enqueue", t, transfer_obj=trig.obj_id, transfer_direction="to_slow")
        for trig in task.prefetch_after:
            src = pool.get((trig.obj_id, BACKING))
            dev = pool.get((trig.obj_id, FAST))
            if dev is not None and dev.state in ("live", "inbound", "reserved"):
                raise SimulationError(f"task {task.id!r} cannot prefetch {trig.obj_id!r}: fast copy exists "
                                      f"(state={dev.state!r})")
            going_out = (dev is not None and dev.state in ("pending_outbound", "outbound")) or \
                        (src is not None and src.state in ("pending_inbound", "inbound"))
            if going_out:
                ref = src if src is not None else dev
                self.deferred.setdefault(trig.obj_id, []).append(
                    _Xfer(trig.obj_id, "from_slow", ref.size,
                          transfer_runtime(ref.size, ch.bandwidth_from_slow, trig.runtime, "from_slow"), ref.type))
                self._note("transfer_deferred", t, transfer_obj=trig.obj_id, transfer_direction="from_slow")
                continue
            if src is None or src.state != "live":
                raise SimulationError(f"task {task.id!r} cannot prefetch {trig.obj_id!r}: no backing source "
                                      f"(state={src.state if src else 'absent'!r})")
            self.queue["from_slow"].append(_Xfer(trig.obj_id, "from_slow", src.size,
                                                 transfer_runtime(src.size, ch.bandwidth_from_slow, trig.runtime, "from_slow"),
                                                 src.type))
            self._note("transfer_enqueue", t, transfer_obj=trig.obj_id, transfer_direction="from_slow")
        self._poke(t)

    def begin(self) -> None:
        """Load the initial objects; the clock is at zero."""
        chain, pool, used = self.chain, self.pool, self.used
        for o in chain.initial_memory:
            if (o.id, o.location) in pool:
                raise SimulationError(f"duplicate ({o.id!r}, {o.location!r}) in initial_memory")
            pool[(o.id, o.location)] = _Entry(o.size, "live", o.type)
            used[o.location] += o.size
        for loc in (FAST, BACKING):
            if self.cap[loc] is not None and used[loc] > self.cap[loc]:
                raise SimulationCapacityError(
                    f"initial memory needs {used[loc]} bytes on {loc}, capacity {self.cap[loc]}",
                    kind="initial", location=loc, capacity_bytes=self.cap[loc],
                    actual_need_bytes=used[loc], overage_bytes=used[loc] - self.cap[loc])
        self.peak_fast, self.peak_backing = used[FAST], used[BACKING]
        self.now = 0.0

    def _run_task(self, idx: int, task: Task) -> float:
        """Wait until the task can start, run it, retire the transfers that end while it runs; returns its end time.
        The task is not settled yet (its outputs are reserved, its directives not applied)."""
        pool, used = self.pool, self.used
        now = self.now
        free_at = now
        need = task.workspace_bytes
        for out in task.outputs:
            if out.location == FAST:
                need += out.size
        self._advance(now)
        while True:
            missing, short = self._blocked_reason(task, need)
            if not missing and not short:
                break
            if task.id not in self.stall_causes:
                self.stall_causes[task.id] = (tuple(missing), bool(short))
            t, d = self._next_completion()
            if d is None:
                if self._on_deadlock(idx, task, now, need, missing):
                    continue
                self._deadlock(task, now, need, missing)
            now = self._complete(d)
        b_need = sum(o.size for o in task.outputs if o.location == BACKING)
        if b_need and self.cap[BACKING] is not None and used[BACKING] + b_need > self.cap[BACKING]:
            raise SimulationCapacityError(
                f"task {task.id!r} cannot allocate {b_need} bytes on backing", kind="backing-output",
                task_id=task.id, location=BACKING, capacity_bytes=self.cap[BACKING],
                actual_need_bytes=used[BACKING] + b_need,
                overage_bytes=used[BACKING] + b_need - self.cap[BACKING])
        for out in task.outputs:
            key = (out.id, out.location)
            if key in pool:
                raise SimulationError(f"task {task.id!r} output {out.id!r} collides with an existing object")
            pool[key] = _Entry(out.size, "reserved", out.type)
            used[out.location] += out.size
        self.workspace = task.workspace_bytes
        if now > free_at:
            self.stalls[task.id] = now - free_at
        else:
            self.stall_causes.pop(task.id, None)
        end = now + task.runtime
        self.intervals.append(TaskInterval(task.id, now, end, "compute"))
        self._note("task_start", now, task_id=task.id)
        # transfers ending at exactly ``end`` retire before the task does
        self._advance(end)
        self.now = end
        return end

    def run(self) -> EventLog:
        self.begin()
        for idx, task in enumerate(self.chain.tasks):
            end = self._run_task(idx, task)
            self._finish_task(idx, task, end)
        return self.finish()

    def finish(self) -> EventLog:
        """Drain the lanes, check the final locations, return the log."""
        chain, pool, used = self.chain, self.pool, self.used
        while True:
            t, d = self._next_completion()
            if d is None:
                break
            self._complete(d)
        if self.queue["from_slow"] or self.queue["to_slow"] or self.deferred:
            raise SimulationCapacityError(
                "transfers still queued at the end of the chain: from_slow="
                f"{[x.obj for x in self.queue['from_slow']]} to_slow={[x.obj for x in self.queue['to_slow']]} "
                f"deferred={sorted(self.deferred)}", kind="stuck-transfers")
        for obj, loc in chain.final_locations.items():
            e = pool.get((obj, loc))
            if e is None or e.state != "live":
                raise SimulationError(f"final location violated: {obj!r} is not live at {loc!r}")
            if loc == BACKING:
                f = pool.get((obj, FAST))
                if f is not None and f.dirty:
                    raise SimulationError(f"final location violated: backing copy of {obj!r} is stale")
        return EventLog(self.intervals, self.events, self.peak_fast, max(self.peak_backing, used[BACKING]),
                        self.trace, self.stalls, self.stall_causes)


def run(chain: TaskChain, validate: bool = True, snapshots: bool = False,
        memory_trace: bool = False) -> EventLog:
    """Simulate an annotated chain.  ``snapshots`` records the event stream."""
    if validate:
        from .validate import validate_chain
        validate_chain(chain)
    try:
        return Simulator(chain, events=snapshots, memory_trace=memory_trace).run()
    except (KeyError, AssertionError) as e:
        # only a chain that the static validator would refuse gets here (validate=False): a directive for a copy that an
        # earlier directive already took away, found when the transfer completes
        raise SimulationError(f"the chain drove the simulation into an inconsistent state ({type(e).__name__}: {e}); "
                              f"validate_chain says what is wrong with it") from e


def compute_lower_bound(chain: TaskChain) -> float:
    """Sum of task runtimes: no plan can finish sooner."""
    return float(sum(t.runtime for t in chain.tasks))
