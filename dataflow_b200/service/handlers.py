"""Verb handlers: store verbs, program registration, ``run`` (bind → execute → capture finals →
fetch), run bookkeeping, misc.  Role parity: reference ``src/dataflow/service/handlers_store.py``,
``handlers_runs.py:22-438`` and ``execution.py:40-426``."""
from __future__ import annotations

import importlib
import threading
import time
from typing import Any

from ..core import (Program, ValidationError, collect_problems, program_content_id, program_from_dict,
                    program_to_dict)
from ..runtime import Buffer, Engine, Session
from ..runtime.trace import trace_to_dict
from .registry import list_resolvers, lookup_resolver
from .wire import ServiceError


class _Env:
    def __init__(self, device, kernel_set):
        self.device, self.kernel_set = device, kernel_set


def _engine(server):
    if getattr(server, "_engine", None) is None:
        server._session = Session(server.backend)
        server._engine = Engine(server.backend, session=server._session, poison_on_free=server.config.poison_on_free)
    return server._engine


def close_engine(server) -> None:
    server._engine = None
    server._session = None
    if server.backend is not None:
        server.backend.synchronize()


def _code_rev() -> str:
    from .. import code_revision
    return code_revision()


def _env_line() -> str:
    from .. import environment_line
    return environment_line()


def install(server) -> None:
    st, H = server.store, server.handlers

    # ------------------------------------------------------------------ misc
    H["health"] = lambda req, p: {"status": "ok", "uptime_s": time.time() - server.state.started}
    H["engine_status"] = lambda req, p: {"backend": server.backend.name(), "device": server.config.device,
                                          "programs": len(server.programs), "runs": len(server.runs),
                                          "counters": dict(server.state.counters), "store": st.query(),
                                          "host_bw_gbs": dict(getattr(server, "host_bw", {})),
                                          "code_rev": _code_rev(), "env": _env_line()}
    H["session_status"] = lambda req, p: {"vendor_allocs": server._session.vendor_allocs()
                                          if getattr(server, "_session", None) else 0}
    def profiler_control(req, p):
        """Open or close the capture window: NVTX ranges of tasks and transfers on / off, and the CUDA profiler API's start /
        stop (what a timeline profiler started with ``--capture-range=cudaProfilerApi`` waits for)."""
        from ..runtime import set_nvtx
        on = req.get("action", "start") in ("start", "on", True)
        set_nvtx(on)
        api = False
        if server.config.device is not None and not server.config.fake:
            try:
                import torch
                (torch.cuda.profiler.start if on else torch.cuda.profiler.stop)()
                api = True
            except Exception:       # noqa: BLE001
                api = False
        return {"nvtx": on, "profiler_api": api}
    H["profiler_control"] = profiler_control
    H["subscribe_events"] = lambda req, p: {"events": server.state.events_since(int(req.get("since", 0)))}
    H["run_events"] = H["subscribe_events"]
    H["list_resolvers"] = lambda req, p: {"resolvers": list_resolvers()}

    def shutdown(req, p):
        server.state.shutdown_requested.set()
        return {}
    H["shutdown"] = shutdown

    def load_plugin(req, p):
        importlib.import_module(req["module"])
        return {"loaded": req["module"]}
    H["load_plugin"] = load_plugin

    # ------------------------------------------------------------------ store verbs
    def put_object(req, payload):
        if payload is None:
            raise ServiceError("BAD_REQUEST", "put_object needs a payload")
        r = st.put(req["id"], payload)
        return {"id": r.id, "size": r.size}
    H["put_object"] = put_object

    def get_object(req, payload):
        r = st.get(req["id"])
        off, n = int(req.get("offset", 0)), int(req.get("size", r.size - int(req.get("offset", 0))))
        if off < 0 or off + n > r.size:
            raise ServiceError("BAD_REQUEST", "slice outside the object")
        return {"id": r.id, "size": r.size}, bytes(st.view(r.id)[off:off + n])
    H["get_object"] = get_object

    def create_object(req, payload):
        r = st.create(req["id"], int(req["size"]), replace=bool(req.get("replace", False)))
        return {"id": r.id, "size": r.size}
    H["create_object"] = create_object

    def materialize_object(req, payload):
        kind = req.get("kind", "zeros")
        r = st.create(req["id"], int(req["size"]), replace=True)
        v = st.view(r.id)
        if kind == "zeros":
            v[:] = bytes(r.size) if r.size < (1 << 24) else b"\0" * r.size
        elif kind == "file":
            with open(req["path"], "rb") as f:
                f.seek(int(req.get("file_offset", 0)))
                data = f.read(r.size)
            if len(data) != r.size:
                raise ServiceError("IO_ERROR", f"{req['path']} holds {len(data)} bytes, wanted {r.size}")
            v[:] = data
        elif kind == "tokens":
            import numpy as np
            rng = np.random.default_rng(int(req.get("seed", 0)))
            v[:] = rng.integers(0, int(req["vocab"]), size=r.size // 4, dtype=np.int32).tobytes()
        else:
            raise ServiceError("BAD_REQUEST", f"unknown materialize kind {kind!r}")
        return {"id": r.id, "size": r.size}
    H["materialize_object"] = materialize_object

    H["release_object"] = lambda req, p: (st.release(req["id"]), {})[1]
    H["protect_object"] = lambda req, p: (st.protect(req["id"], True), {})[1]
    H["unprotect_object"] = lambda req, p: (st.protect(req["id"], False), {})[1]
    H["duplicate_object"] = lambda req, p: {"size": st.duplicate(req["src"], req["dst"]).size}
    H["wipe"] = lambda req, p: {"released": st.wipe(req.get("scope", "unprotected"), bool(req.get("force", False)))}
    H["query_object"] = lambda req, p: (lambda r: {"id": r.id, "size": r.size, "protected": r.protected, "leases": r.leases})(st.get(req["id"]))
    H["list_objects"] = lambda req, p: {"objects": [{"id": r.id, "size": r.size, "protected": r.protected}
                                                     for r in sorted(st.objects.values(), key=lambda r: r.id)]}
    H["query_backing"] = lambda req, p: st.query()
    H["query_fast"] = lambda req, p: {"fast_slab_bytes": server._session.native.fast_slab()[1]
                                      if getattr(server, "_session", None) else 0}

    # ------------------------------------------------------------------ programs
    def register_program(req, payload):
        d = req["program"]
        try:
            prog = program_from_dict(d)
        except (KeyError, ValueError) as e:
            raise ServiceError("BAD_REQUEST", f"program does not parse: {e}") from None
        probs = collect_problems(prog)
        if probs:
            raise ServiceError("BAD_REQUEST", "invalid program", problems=probs[:20])
        pid = program_content_id(program_to_dict(prog))
        if req.get("expect_prog_id") and req["expect_prog_id"] != pid:
            raise ServiceError("VERSION_SKEW", f"client expected {req['expect_prog_id']}, server computed {pid}")
        entry = {"program": prog, "resolver_spec": req.get("resolver_spec"), "registered": time.time(),
                 "host": bool(prog.tasks and prog.tasks[0].host), "runs": 0, "placement": None}
        out = {"prog_id": pid, "tasks": len(prog.tasks), "host": entry["host"]}
        if req.get("prepare_placement") and not entry["host"]:
            # dry run on the virtual-time backend: every fast allocation of a run gets an offset ahead of time; the extent says
            # how much pool the program needs when nothing fragments (refused here, not at run time, when it cannot fit)
            out["placement"] = prepare_placement(entry, req.get("placement_capacity"))
        server.programs[pid] = entry
        server.state.emit("program_registered", prog_id=pid, name=prog.name)
        return out
    H["register_program"] = register_program

    def prepare_placement(entry, capacity=None) -> dict:
        from ..runtime.placement import PlacementError, peak_live_bytes, plan_placement
        prog = entry["program"]
        cap = int(capacity) if capacity else (int(prog.fast_memory_capacity) if prog.fast_memory_capacity else None)
        try:
            pl = plan_placement(prog, cap)
        except PlacementError as e:
            raise ServiceError("BAD_REQUEST", f"no static placement fits: {e}") from None
        entry["placement"] = pl
        return {"extent_bytes": int(pl.top), "peak_live_bytes": int(peak_live_bytes(pl.lifetimes)), "allocations": len(pl.lifetimes),
                "capacity": cap}

    def validate_program(req, payload):
        try:
            probs = collect_problems(program_from_dict(req["program"]))
        except (KeyError, ValueError) as e:
            probs = [str(e)]
        return {"valid": not probs, "problems": probs}
    H["validate_program"] = validate_program

    def unregister_program(req, payload):
        if server.programs.pop(req["prog_id"], None) is None:
            raise ServiceError("UNKNOWN_PROGRAM", req["prog_id"])
        return {}
    H["unregister_program"] = unregister_program
    H["list_programs"] = lambda req, p: {"programs": [{"prog_id": k, "name": v["program"].name, "runs": v["runs"]}
                                                       for k, v in server.programs.items()]}

    # ------------------------------------------------------------------ run
    def run(req, payload):
        pid = req["prog_id"]
        entry = server.programs.get(pid)
        if entry is None:
            raise ServiceError("UNKNOWN_PROGRAM", pid)
        prog: Program = entry["program"]
        args = dict(req.get("args") or {})
        # lease pre-pass: a snapshot is still copying one of the objects this run touches
        touched = {o.id for o in prog.initial_objects}
        leased = st.leased(touched)
        if leased:
            raise ServiceError("LEASED", f"objects leased by a snapshot: {leased[:4]}", park=True)
        initial: dict[str, Buffer] = {}
        missing, mismatch = [], []
        for o in prog.initial_objects:
            r = st.objects.get(o.id)
            if r is None:
                missing.append(o.id)
            elif r.size != o.size_bytes:
                mismatch.append((o.id, r.size, o.size_bytes))
            else:
                initial[o.id] = Buffer(st.address(o.id), r.size, "backing", o.id)
        if missing:
            raise ServiceError("MISSING_INPUTS", f"store lacks {missing[:6]}", missing=missing)
        if mismatch:
            raise ServiceError("BINDING_MISMATCH", f"size mismatch (id, store, program): {mismatch[:4]}")
        rid = server.state.new_id("r")
        rec = {"run_id": rid, "prog_id": pid, "state": "running", "started": time.time(), "args": args}
        server.runs[rid] = rec
        server.state.emit("run_started", run_id=rid, prog_id=pid)
        cancel = threading.Event()
        server.cancel_events[rid] = cancel
        resolver = lookup_resolver(entry["resolver_spec"], _Env(server.config.device, server.config.kernel_set))
        st.begin_created_log()
        try:
            if entry["host"]:
                _execute_host(server, prog, resolver, args)
                result = None
            else:
                # landing extents for final backing objects the program creates (losses, checkpoints of activations)
                sizes = prog.object_sizes()
                for oid, loc in prog.final_locations.items():
                    if loc == "backing" and oid not in initial:
                        r = st.create(oid, sizes[oid], replace=True)
                        initial[oid] = Buffer(st.address(oid), r.size, "backing", oid)
                groups = server.nm.group_handles() if server.nm is not None else {}
                placement = entry.get("placement") if req.get("use_placement", True) else None
                eng = _engine(server)
                if placement is not None:
                    # planned offsets need a pool that reaches them: the extent of the packing (a program without a capacity of
                    # its own would otherwise run on exact-size vendor allocations, where offsets mean nothing)
                    server._session.native.ensure_pools(int(placement.top) + (1 << 20), 0, 0.0)
                result = eng.execute(prog, resolver, initial, run_args=args, groups=groups,
                                                 cancel_event=cancel,
                                                 placement=placement)
                if result.outcome.kind.value == "SUCCESS":
                    for oid, b in result.finals.items():
                        if b.location == "backing" and oid in st.objects and b.ptr != st.address(oid):
                            import ctypes
                            ctypes.memmove(st.address(oid), b.ptr, min(b.size, st.get(oid).size))   # capture finals
        except ServiceError:
            st.rollback_created()
            rec.update(state="failed", finished=time.time())
            raise
        except Exception as e:      # noqa: BLE001
            st.rollback_created()
            rec.update(state="failed", finished=time.time(), message=str(e))
            server.state.emit("run_failed", run_id=rid)
            raise ServiceError("RUN_FAILED", f"{type(e).__name__}: {e}", run_id=rid) from None
        finally:
            server.cancel_events.pop(rid, None)
        if result is not None and not result.outcome.ok:
            st.rollback_created()
            kind = result.outcome.kind.value
            rec.update(state="cancelled" if kind == "CANCELLED" else "failed", finished=time.time(),
                       message=result.outcome.message, task_id=result.outcome.task_id)
            server.state.emit("run_failed", run_id=rid)
            raise ServiceError("CANCELLED" if kind == "CANCELLED" else "RUN_FAILED", result.outcome.message,
                               run_id=rid, task_id=result.outcome.task_id, traceback=result.outcome.traceback[-1500:])
        st.end_created_log()
        entry["runs"] += 1
        out: dict[str, Any] = {"run_id": rid, "state": "done"}
        if result is not None:
            rec.update(makespan_us=result.makespan_us, peak_fast_bytes=result.peak_fast_bytes,
                       slab_overflows=result.slab_overflows, pressure_evictions=result.pressure_evictions,
                       placement_escapes=result.placement_escapes)
            out.update(makespan_us=result.makespan_us, peak_fast_bytes=result.peak_fast_bytes,
                       slab_overflows=result.slab_overflows, placement_escapes=result.placement_escapes)
            if req.get("trace"):
                out["trace"] = trace_to_dict(result.trace)
            rec["trace"] = result.trace
        fetched = {}
        import struct
        for oid in req.get("fetch") or ():
            if oid in st.objects and st.get(oid).size == 4:
                fetched[oid] = struct.unpack("<f", bytes(st.view(oid)[:4]))[0]
        out["fetched"] = fetched
        rec.update(state="done", finished=time.time())
        server.state.emit("run_done", run_id=rid)
        return out
    H["run"] = run

    def cancel_run(req, payload):
        ev = server.cancel_events.get(req.get("run_id", ""))
        if ev is None:
            for ev in server.cancel_events.values():      # no id: cancel whatever is running
                ev.set()
            return {"cancelled": bool(server.cancel_events)}
        ev.set()
        return {"cancelled": True}
    H["cancel_run"] = cancel_run

    def run_status(req, payload):
        rec = server.runs.get(req["run_id"])
        if rec is None:
            raise ServiceError("UNKNOWN_RUN", req["run_id"])
        return {k: v for k, v in rec.items() if k != "trace"}
    H["run_status"] = run_status
    H["list_runs"] = lambda req, p: {"runs": [{k: v for k, v in r.items() if k != "trace"} for r in server.runs.values()]}

    def export_trace(req, payload):
        rec = server.runs.get(req["run_id"])
        if rec is None or "trace" not in rec:
            raise ServiceError("UNKNOWN_RUN", req.get("run_id", ""))
        return {"trace": trace_to_dict(rec["trace"])}
    H["export_trace"] = export_trace


def _execute_host(server, prog: Program, resolver, args) -> None:
    """HOST tasks run on the dispatcher thread over the store's backing extents (no streams, no events)."""
    from ..runtime.executable import TaskContext
    st = server.store
    if resolver is None:
        raise ServiceError("BAD_REQUEST", "host program registered without a resolver spec")
    for t in prog.tasks:
        bufs = tuple(Buffer(st.address(i), st.get(i).size, "backing", i) for i in t.inputs)
        ctx = TaskContext(task=t, stream=0, inputs=bufs, outputs=(), backend=server.backend, run_args=args)
        resolver(t).launch(ctx)
