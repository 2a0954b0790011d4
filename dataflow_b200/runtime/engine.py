"""Python face of the native task executor.

``Engine(backend).execute(program, resolver, ...)`` compiles the Program to the
executor's index form, runs the C++ dispatch loop (GIL released; it is taken
back only to call ``Executable.launch``) and returns a ``RunResult`` with the
outcome, the interval trace and the health counters.  API parity: reference
``src/dataflow/runtime/engine.py:399-506`` and ``docs/engine_api.md:9-85``.
"""
from __future__ import annotations

import enum
import threading
from dataclasses import dataclass, field
from typing import Any, Callable, Mapping

from ..core import Program, validate_program
from . import _runtime as _rt
from .executable import Buffer, Executable, TaskContext
from .trace import Interval, RunTrace, TraceEvent

FAST, BACKING = 0, 1
_LOC = {"fast": FAST, "backing": BACKING}


class RunOutcomeKind(str, enum.Enum):
    SUCCESS = "SUCCESS"
    FAILED = "FAILED"
    CANCELLED = "CANCELLED"


@dataclass
class RunOutcome:
    kind: RunOutcomeKind
    message: str = ""
    task_id: str = ""
    error_kind: str = ""
    traceback: str = ""

    @property
    def ok(self) -> bool:
        return self.kind is RunOutcomeKind.SUCCESS


class ExecutionError(RuntimeError):
    pass


class DeadlockError(ExecutionError):
    pass


ENGINE_INVARIANT_ERRORS = ("LedgerError", "ExecutionError", "FinalLocationError", "BindingMismatch")


@dataclass
class RunResult:
    outcome: RunOutcome
    trace: RunTrace
    makespan_us: float
    peak_fast_bytes: int
    peak_backing_bytes: int
    slab_overflows: int
    pressure_evictions: int
    placement_escapes: int
    vendor_allocs: int
    stats: dict[str, Any]
    finals: dict[str, Buffer] = field(default_factory=dict)

    def raise_if_failed(self) -> "RunResult":
        if self.outcome.kind is RunOutcomeKind.FAILED:
            cls = DeadlockError if self.outcome.error_kind == "DeadlockError" else ExecutionError
            raise cls(f"[{self.outcome.error_kind}] {self.outcome.message}"
                      + (f" (task {self.outcome.task_id})" if self.outcome.task_id else "")
                      + (("\n" + self.outcome.traceback) if self.outcome.traceback else ""))
        return self

    def close(self) -> None:
        pass


class Session:
    """Streams and buffer pools that live across ``execute`` calls."""

    def __init__(self, backend):
        self.backend = backend
        self.native = _rt.Session(backend)

    def vendor_allocs(self) -> int:
        return self.native.vendor_allocs()

    def compute_stream_handle(self) -> int:
        return self.backend.stream_handle(self.native.compute_stream)

    def resident(self) -> dict[str, tuple[int, int]]:
        """``{object id: (device address, bytes)}`` of the final-fast objects held since the last run."""
        return dict(self.native.resident())

    def drop_resident(self) -> None:
        self.native.drop_resident()


class ChainIndex:
    """Program → executor index form, cached per program object."""

    def __init__(self, program: Program):
        ir = _rt.ProgramIR()
        ir.name = program.name
        ir.fast_cap = -1 if program.fast_memory_capacity is None else int(program.fast_memory_capacity)
        ir.backing_cap = -1 if program.backing_memory_capacity is None else int(program.backing_memory_capacity)
        ir.bw_from = int(program.bandwidth_from_slow or 0)
        ir.bw_to = int(program.bandwidth_to_slow or 0)
        index: dict[str, int] = {}
        objs: list[Any] = []
        # planned programs budget task scratch outside the object pool (see lowering.planning)
        ext_ws = (program.metadata or {}).get("workspace_accounting") == "external"

        def obj(oid: str, size: int):
            if oid not in index:
                o = _rt.ObjIR()
                o.id, o.size = oid, int(size)
                index[oid] = len(objs)
                objs.append(o)
            return objs[index[oid]]

        for o in program.initial_objects:
            rec = obj(o.id, o.size_bytes)
            if o.location == "fast":
                rec.init_fast = True
            else:
                rec.init_backing = True
        for t in program.tasks:
            for out in t.outputs:
                obj(out.id, out.size_bytes)
        for ti, t in enumerate(program.tasks):
            for i in t.inputs:
                objs[index[i]].last_ref = ti
            for d in t.offload_after:
                objs[index[d.object_id]].last_ref = ti
            for d in t.prefetch_after:
                objs[index[d.object_id]].last_ref = ti
        for oid, loc in program.final_locations.items():
            objs[index[oid]].final_loc = _LOC[loc]
        for o in objs:
            ir.add_obj(o)
        for t in program.tasks:
            tr = _rt.TaskIR()
            tr.id = t.id
            tr.inputs = [index[i] for i in t.inputs]
            tr.mutates = [index[i] for i in t.mutates]
            tr.releases = [index[i] for i in t.releases_after]
            tr.runtime_us = float(t.runtime_us)
            tr.workspace = 0 if ext_ws else int(t.workspace_bytes)
            for out in t.outputs:
                tr.add_output(index[out.id], _LOC[out.location])
            for d in t.offload_after:
                tr.add_offload(index[d.object_id], -1.0 if d.runtime_us is None else float(d.runtime_us))
            for d in t.prefetch_after:
                tr.add_prefetch(index[d.object_id], -1.0 if d.runtime_us is None else float(d.runtime_us))
            ir.add_task(tr)
        self.ir = ir
        self.index = index
        self.ir_object_ids = [o.id for o in objs]
        self.program = program


class Engine:
    def __init__(self, backend, validate: bool = True, strict_final_locations: bool = True,
                 poison_on_free: bool = False, session: Session | None = None):
        self.backend = backend
        self.validate = validate
        self.strict_final_locations = strict_final_locations
        self.poison_on_free = poison_on_free
        self.session = session or Session(backend)
        self._native = _rt.Engine(self.session.native)
        self._index_cache: dict[int, ChainIndex] = {}

    def chain_index(self, program: Program) -> ChainIndex:
        ci = self._index_cache.get(id(program))
        if ci is None or ci.program is not program:
            if self.validate:
                validate_program(program)
            ci = ChainIndex(program)
            self._index_cache[id(program)] = ci
            if len(self._index_cache) > 16:
                self._index_cache.pop(next(iter(self._index_cache)))
        return ci

    def execute(self, program: Program, resolver: Callable | None = None,
                initial_buffers: Mapping[str, Buffer] | None = None, *,
                run_args: Mapping[str, Any] | None = None, groups: Mapping[str, Any] | None = None,
                cancel_event: threading.Event | None = None, record_events: bool = False,
                slab_headroom: float = 0.0, manage_pools: bool = True, keep_resident: bool = False,
                dispatch_ahead: int = 0, record_allocs: bool = False, placement=None, annotator=None,
                annotate_rename: Callable[[str, str], str] | None = None) -> RunResult:
        """``placement``: a ``runtime.placement.Placement`` for this program (static offsets of every fast allocation);
        ``record_allocs`` returns the allocation log the placement is computed from (``result.stats["allocs"]``).
        ``annotator`` (``runtime.annotate``; default: what ``DATAFLOW_ANNOTATE`` names) is told every task launch and
        transfer issue as a range; ``annotate_rename(name, kind)`` gives the displayed names only."""
        from .annotate import annotator_from_env, make_hook
        hook = make_hook(annotator if annotator is not None else annotator_from_env(), annotate_rename)
        ci = self.chain_index(program)
        tasks = program.tasks
        run_values: dict[str, Any] = {}
        failure: dict[str, str] = {}
        launch = None
        if resolver is not None:
            exes = [resolver(t) for t in tasks]
            backend = self.backend
            run_args = dict(run_args or {})
            groups = dict(groups or {})

            def launch(idx, in_ptrs, out_ptrs, stream):      # called from the executor thread with the GIL
                t = tasks[idx]
                ctx = TaskContext(
                    task=t, stream=stream,
                    inputs=tuple(Buffer(p, ci.ir_sizes[i], "fast", i) for p, i in zip(in_ptrs, t.inputs)),
                    outputs=tuple(Buffer(p, o.size_bytes, o.location, o.id) for p, o in zip(out_ptrs, t.outputs)),
                    backend=backend, run_args=run_args, run_values=run_values, groups=groups)
                try:
                    exes[idx].launch(ctx)
                except BaseException:
                    import traceback
                    failure["traceback"] = traceback.format_exc()
                    raise
            if not hasattr(ci, "ir_sizes"):
                ci.ir_sizes = program.object_sizes()
        initial = {}
        for oid, b in (initial_buffers or {}).items():
            initial[oid] = (int(b.ptr), int(b.size), _LOC[b.location])
        cancel = None
        watcher = None
        if cancel_event is not None:
            cancel = _rt.CancelFlag()
            stop = threading.Event()

            def _watch():
                while not stop.is_set():
                    if cancel_event.wait(0.01):
                        cancel.set()
                        return
            watcher = threading.Thread(target=_watch, daemon=True)
            watcher.start()
        try:
            raw = self._native.execute(ci.ir, launch, initial, self.strict_final_locations,
                                       self.poison_on_free, record_events, slab_headroom, cancel, manage_pools,
                                       keep_resident, int(dispatch_ahead), bool(record_allocs),
                                       placement.for_index(ci) if placement is not None else [], hook)
        finally:
            if watcher is not None:
                stop.set()
        st = raw["stats"]
        waits = run_values.get("_comm_waits")
        if waits:
            # device-timed stalls of the compute stream on transfers issued on another stream (both events have fired:
            # the run is complete)
            st = dict(st)
            try:
                st["exposed_comm_us"] = 1e3 * sum(max(a.elapsed_time(b), 0.0) for a, b in waits)
                st["comm_waits"] = len(waits)
            except RuntimeError:
                pass
        trace = RunTrace([Interval(n, tr, a, b) for n, tr, a, b in raw["intervals"]],
                         [TraceEvent(k, w, f) for k, w, f in raw["events"]],
                         st["peak_fast_bytes"], st["peak_backing_bytes"])
        outcome = RunOutcome(RunOutcomeKind(raw["outcome"]), raw["message"], raw["failed_task"],
                             raw["error_kind"], failure.get("traceback", ""))
        finals = {k: Buffer(v[1], v[2], "fast" if v[0] == FAST else "backing", k) for k, v in raw["finals"].items()}
        if record_allocs:
            st = dict(st)
            st["allocs"] = [(ci.ir_object_ids[o] if o >= 0 else None, size, ptr, kind) for o, size, ptr, kind in raw["allocs"]]
        return RunResult(outcome, trace, st["makespan_us"], st["peak_fast_bytes"], st["peak_backing_bytes"],
                         st["slab_overflows"], st["pressure_evictions"], st["placement_escapes"],
                         st["vendor_allocs"], dict(st), finals)
