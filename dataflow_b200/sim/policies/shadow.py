"""Shadow: the simulator as a state machine a planner steps, questions, amends and forks.

``Simulator.run`` plays a finished plan from start to end.  A planner that decides as it goes needs the same machine one
task at a time, with the plan still open:

    sh = Shadow(bare_chain, capacity)
    while not sh.done:
        sh.step()                       # wait for operands and room, run the next task, settle it (outputs live)
        ...                             # look: sh.now, sh.fast_used, sh.resident(), sh.where(obj), sh.eta(obj), sh.lane_clear(..)
        sh.release(obj); sh.offload(obj); sh.prefetch(obj)      # directives of the task that just ended
        sh.commit()                     # apply them: releases free at once, transfers join their lanes
    planned, log = sh.result()

``fork()`` copies the whole state, so a planner can try a decision, run ahead (``lookahead(k)``) and throw the copy away; the
reactive planner uses that to learn whether the next task can start at all before it closes a boundary.  The semantics
are the simulator's own (``Shadow`` subclasses it and reuses its lanes, ledger and directive rules), so the chain a shadow
run leaves behind replays to the same event log.
Reference role: ``src/dataflow_sim/policies/shadow.py`` (``ShadowSimulator``: queries and mutators on a mirrored state).
"""
from __future__ import annotations

from dataclasses import replace

from ..errors import SimulationCapacityError, SimulationError
from ..schema import Task, TaskChain, TransferTrigger
from ..simulator import BACKING, FAST, Simulator, _Entry, _Xfer, transfer_runtime


def _open_task(t: Task) -> Task:
    return replace(t, releases_after=list(t.releases_after), offload_after=list(t.offload_after),
                   prefetch_after=list(t.prefetch_after))


class Shadow(Simulator):
    def __init__(self, chain: TaskChain, capacity: int | None = None, *, initial=None):
        cap = capacity if capacity is not None else chain.fast_memory_capacity
        work = replace(chain, tasks=[_open_task(t) for t in chain.tasks], fast_memory_capacity=cap,
                       initial_memory=list(initial if initial is not None else chain.initial_memory))
        super().__init__(work)
        self.idx = 0                     # the next task to run
        self.open: Task | None = None    # the task that has ended and whose directives are being decided
        self.begin()

    # ------------------------------------------------------------------------------------------------------------ stepping
    @property
    def done(self) -> bool:
        return self.idx >= len(self.chain.tasks) and self.open is None

    def step(self) -> Task:
        """Run the next task to its end and settle it.  Its directives are open until ``commit``."""
        if self.open is not None:
            raise SimulationError("commit the open task before stepping")
        task = self.chain.tasks[self.idx]
        end = self._run_task(self.idx, task)
        self._settle_task(self.idx, task, end)
        self.open = task
        return task

    def commit(self) -> None:
        task = self.open
        if task is None:
            raise SimulationError("no open task to commit")
        self._apply_directives(self.idx, task, self.now)
        self.open = None
        self.idx += 1

    def result(self):
        """(annotated chain, event log) once every task has been stepped and committed."""
        if not self.done:
            raise SimulationError("the shadow run is not finished")
        return self.chain, self.finish()

    # ----------------------------------------------------------------------------------------------------------- directives
    def _need_open(self) -> Task:
        if self.open is None:
            raise SimulationError("directives can be added only between step() and commit()")
        return self.open

    def release(self, obj: str) -> None:
        self._need_open().releases_after.append(obj)

    def offload(self, obj: str) -> None:
        self._need_open().offload_after.append(TransferTrigger(obj))

    def prefetch(self, obj: str) -> None:
        self._need_open().prefetch_after.append(TransferTrigger(obj))

    def retract(self) -> None:
        """Drop the directives added to the open task so far."""
        t = self._need_open()
        t.releases_after.clear()
        t.offload_after.clear()
        t.prefetch_after.clear()

    # -------------------------------------------------------------------------------------------------------------- queries
    @property
    def fast_used(self) -> int:
        return self.used[FAST]

    @property
    def fast_free(self) -> float:
        return self._free(FAST)

    def where(self, obj: str) -> tuple[str | None, str | None]:
        """(state of the fast copy, state of the backing copy); None where there is no copy."""
        f, b = self.pool.get((obj, FAST)), self.pool.get((obj, BACKING))
        return (f.state if f else None), (b.state if b else None)

    def resident(self) -> dict[str, _Entry]:
        """The live fast copies (not in flight either way)."""
        return {k[0]: e for k, e in self.pool.items() if k[1] == FAST and e.state == "live"}

    def needs_offload(self, obj: str) -> bool:
        """True when dropping the fast copy would lose bytes: it is dirty, or there is no live backing copy."""
        f, b = self.pool.get((obj, FAST)), self.pool.get((obj, BACKING))
        return f is not None and (f.dirty or b is None or b.state != "live")

    def queued(self, direction: str) -> list[str]:
        out = [x.obj for x in self.queue[direction]]
        if direction == "from_slow":
            out += [x.obj for xs in self.deferred.values() for x in xs]
        return out

    def lane_clear(self, direction: str) -> float:
        """When the lane will have moved everything it has now, if nothing blocks it (a lower bound)."""
        fl = self.flight[direction]
        t = fl.end if fl is not None else self.now
        return t + sum(x.runtime for x in self.queue[direction])

    def eta(self, obj: str) -> float | None:
        """When the object will be live in fast memory: now if it is, the lane's estimate if a fetch is under way or
        queued, None if nobody has asked for it."""
        f = self.pool.get((obj, FAST))
        if f is not None and f.state == "live":
            return self.now
        fl = self.flight["from_slow"]
        t = fl.end if fl is not None else self.now
        if fl is not None and fl.obj == obj:
            return t
        for x in self.queue["from_slow"]:
            t += x.runtime
            if x.obj == obj:
                return t
        if obj in self.deferred:
            return max(t, self.lane_clear("to_slow")) + self.deferred[obj][0].runtime
        return None

    def fetch_time(self, obj: str) -> float:
        e = self.pool.get((obj, BACKING)) or self.pool.get((obj, FAST))
        return transfer_runtime(e.size, self.chain.bandwidth_from_slow, None, "from_slow")

    def offload_time(self, obj: str) -> float:
        e = self.pool.get((obj, FAST))
        return transfer_runtime(e.size, self.chain.bandwidth_to_slow, None, "to_slow")

    # -------------------------------------------------------------------------------------------------------------- forking
    def fork(self, depth: int | None = None) -> "Shadow":
        """An independent copy.  ``depth``: how many tasks from the current one on get their own directive lists (all by
        default; a short probe needs only the few it will run)."""
        c = object.__new__(Shadow)
        c.__dict__.update(self.__dict__)
        c.pool = {k: _Entry(e.size, e.state, e.type, e.dirty) for k, e in self.pool.items()}
        c.used = dict(self.used)
        cp = lambda x: None if x is None else _Xfer(x.obj, x.direction, x.size, x.runtime, x.type, x.start, x.end)
        c.queue = {d: [cp(x) for x in q] for d, q in self.queue.items()}
        c.flight = {d: cp(x) for d, x in self.flight.items()}
        c.deferred = {o: [cp(x) for x in xs] for o, xs in self.deferred.items()}
        c.seq = dict(self.seq)
        c.intervals = list(self.intervals)
        c.events = list(self.events)
        c.trace = list(self.trace)
        c.stalls = dict(self.stalls)
        c.stall_causes = dict(self.stall_causes)
        tasks = list(self.chain.tasks)
        for j in range(self.idx, len(tasks) if depth is None else min(self.idx + depth, len(tasks))):
            tasks[j] = _open_task(tasks[j])
        c.chain = replace(self.chain, tasks=tasks)
        c.open = tasks[self.idx] if self.open is not None else None
        return c

    def lookahead(self, tasks_ahead: int = 1):
        """On a fork: commit the open task as it stands and run ``tasks_ahead`` more tasks with whatever directives they
        carry.  Returns ``(stall_us, None)``, or ``(None, error)`` when the run cannot go on."""
        c = self.fork(tasks_ahead + 1)
        try:
            if c.open is not None:
                c.commit()
            before = sum(c.stalls.values())
            for _ in range(tasks_ahead):
                if c.idx >= len(c.chain.tasks):
                    break
                c.step()
                c.commit()
            return sum(c.stalls.values()) - before, None
        except (SimulationCapacityError, SimulationError) as e:
            return None, e
