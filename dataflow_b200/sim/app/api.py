"""HTTP API of the simulator: presets, plan-free previews, and planned + simulated steps.

    GET  /api/health               liveness + version
    GET  /api/presets              hardware rows, model library, policies
    POST /api/workloads/preview    model (by name or explicit program) + training config + hardware -> totals, no plan
    POST /api/simulate             same input + memory budget + policy -> plan, simulate, summary, timelines; on request
                                   (``panels``) the annotated plan, memory by object type, residency spans for the event
                                   scrubber, the stall report, the first-touch tape and the planner's candidate table
    POST /api/compare              the same workload planned by several policies, one row each
    POST /api/sweep                the same workload and policy over a list of budgets
    POST /api/validate             a task chain (JSON) -> the static validator's problems, by stage

Reference role: ``src/dataflow_sim/app/server/main.py:78-211`` (request models), ``:216,221,346,552`` (the four routes).
``GET /`` serves a single-page front end (``static/index.html``: inputs, summary, compute / copy timeline with an event
scrubber, device memory by object type, time by phase and by kind of op, the most expensive ops, the annotated plan, the
stall report, the planner's candidates, the first-touch tape, planner comparison, budget sweep, measured-run overlay from a
trace file — plain JavaScript and SVG over these routes, panel data computed in ``views.py``; the reference's is a React app).
"""
from __future__ import annotations

from typing import Any

import os

from fastapi import FastAPI, HTTPException
from fastapi.responses import HTMLResponse
from pydantic import BaseModel, Field

from ..policies import get_all_policies
from ..simulator import run as simulate
from ..workloads import (HARDWARE_PRESETS, MODEL_LIBRARY, DTypePolicy, HardwareSpec, ParallelismConfig, TrainingConfig, WorkloadProgram,
                         compute_summary, get_hardware, get_model, preview_workload, realize_workload, trace_training_model)

VERSION = "1"


class TrainingRequest(BaseModel):
    seq_len: int = 4096
    tokens_per_round: int = 16384
    rounds: int = 1
    optimizer: str = "adamw"
    optimizer_placement: str = "interleaved"
    recompute: str = "none"
    dtypes: dict[str, Any] = Field(default_factory=dict)
    parallel: dict[str, int] = Field(default_factory=dict)

    def config(self) -> TrainingConfig:
        return TrainingConfig(self.seq_len, self.tokens_per_round, self.rounds, self.optimizer, self.optimizer_placement,
                              self.recompute, DTypePolicy(**self.dtypes), ParallelismConfig(**self.parallel))


class WorkloadRequest(BaseModel):
    model: str | None = None                          # a name from the library ...
    program: dict[str, Any] | None = None             # ... or an explicit dataflow-workload/v1 program
    training: TrainingRequest = Field(default_factory=TrainingRequest)
    hardware: str = "B200"
    hardware_overrides: dict[str, Any] = Field(default_factory=dict)


class SimulateRequest(WorkloadRequest):
    fast_memory_gib: float | None = None
    policy: str = "pressurefit"
    policy_args: dict[str, Any] = Field(default_factory=dict)
    timeline: bool = True
    memory_trace: bool = False
    panels: list[str] = Field(default_factory=list)   # any of: plan, memory_by_type, residency, stalls, references, candidates


class CompareRequest(SimulateRequest):
    policies: list[str] = Field(default_factory=list)   # empty = every registered policy


class SweepRequest(SimulateRequest):
    budgets_gib: list[float] = Field(default_factory=list)


class ValidateRequest(BaseModel):
    chain: dict[str, Any]
    planning_input: bool = False                       # check as a planner's input (bare chain) instead of a finished plan


def _hardware(req: WorkloadRequest) -> HardwareSpec:
    try:
        hw = get_hardware(req.hardware)
    except KeyError as e:
        raise HTTPException(status_code=404, detail=str(e)) from e
    if req.hardware_overrides:
        from dataclasses import replace
        for k, v in req.hardware_overrides.items():
            if isinstance(v, (int, float)) and not isinstance(v, bool) and v < 0:
                raise HTTPException(status_code=422, detail=f"bad hardware override: {k} = {v} is negative")
        try:
            hw = replace(hw, **req.hardware_overrides)
        except TypeError as e:
            raise HTTPException(status_code=422, detail=f"bad hardware override: {e}") from e
    return hw


def _program(req: WorkloadRequest) -> WorkloadProgram:
    if (req.model is None) == (req.program is None):
        raise HTTPException(status_code=422, detail="give exactly one of `model` and `program`")
    if req.program is not None:
        try:
            return WorkloadProgram.model_validate(req.program)
        except ValueError as e:
            raise HTTPException(status_code=422, detail=str(e)) from e
    try:
        return trace_training_model(get_model(req.model), req.training.config())
    except KeyError as e:
        raise HTTPException(status_code=404, detail=str(e)) from e
    except (TypeError, ValueError) as e:
        raise HTTPException(status_code=422, detail=str(e)) from e


def create_app() -> FastAPI:
    app = FastAPI(title="dataflow_b200 simulator", version=VERSION)

    @app.get("/", response_class=HTMLResponse)
    def index():
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "static", "index.html"), encoding="utf-8") as f:
            return f.read()

    @app.get("/api/health")
    def health():
        return {"ok": True, "version": VERSION}

    @app.get("/api/presets")
    def presets():
        return {"hardware": {k: v.to_dict() for k, v in HARDWARE_PRESETS.items()},
                "models": {k: {"d_model": m.d_model, "n_layers": m.n_layers, "vocab": m.vocab} for k, m in MODEL_LIBRARY.items()},
                "policies": sorted(get_all_policies()),
                "recompute": ["none", "selective", "full"], "optimizers": ["adamw", "muon", "sgdm", "sgd", "frozen"]}

    @app.post("/api/workloads/preview")
    def preview(req: WorkloadRequest):
        hw = _hardware(req)
        prog = _program(req)
        try:
            return {"preview": preview_workload(prog, hw), "metadata": prog.metadata}
        except ValueError as e:
            raise HTTPException(status_code=422, detail=str(e)) from e

    def _plan(req: SimulateRequest, policy: str, cap: int | None, prog, hw):
        """(planned chain, planner's own result object or None)."""
        policies = get_all_policies()
        if policy not in policies:
            raise HTTPException(status_code=404, detail=f"unknown policy {policy!r}; known: {sorted(policies)}")
        chain = realize_workload(prog, hw, cap)
        if policy in ("pressurefit", "lookahead") and not req.policy_args:
            from ..policies.lookahead import lookahead
            from ..policies.pressurefit import pressurefit
            res = (pressurefit if policy == "pressurefit" else lookahead)(chain, chain.fast_memory_capacity)
            return res.chain, res
        return policies[policy](chain, chain.fast_memory_capacity, **req.policy_args), None

    def _cap(gib: float | None) -> int | None:
        return int(gib * (1 << 30)) if gib is not None else None

    @app.post("/api/simulate")
    def simulate_route(req: SimulateRequest):
        from . import views
        hw = _hardware(req)
        prog = _program(req)
        want = set(req.panels)
        unknown = want - {"plan", "memory_by_type", "residency", "stalls", "references", "candidates"}
        if unknown:
            raise HTTPException(status_code=422, detail=f"unknown panels {sorted(unknown)}")
        try:
            planned, result = _plan(req, req.policy, _cap(req.fast_memory_gib), prog, hw)
            log = simulate(planned, memory_trace=req.memory_trace, snapshots=bool(want & {"memory_by_type", "residency"}))
        except HTTPException:
            raise
        except Exception as e:                      # planner / simulator refusals are the caller's answer, not a crash
            raise HTTPException(status_code=422, detail=f"{type(e).__name__}: {e}") from e
        out: dict[str, Any] = {"summary": compute_summary(planned, log, prog, hw), "preview": preview_workload(prog, hw),
                               "policy": req.policy, "metadata": prog.metadata}
        if req.timeline:
            out["timeline"] = [{"id": iv.task_id, "track": iv.track, "start": iv.start, "end": iv.end} for iv in log.task_intervals]
        if req.memory_trace:
            out["memory_trace"] = [{"t": p.t, "fast_bytes": p.fast_bytes, "workspace_bytes": p.workspace_bytes} for p in log.memory_trace]
        if "plan" in want:
            out["plan"] = views.plan_table(planned, log)
        if "memory_by_type" in want:
            out["memory_by_type"] = views.memory_by_type(planned, log)
        if "residency" in want:
            sizes = planned.sizes()
            types = {o.id: o.type for o in planned.initial_memory}
            types.update({o.id: o.type for t in planned.tasks for o in t.outputs})
            out["residency"] = [{"id": o, "bytes": sizes.get(o, 0), "type": types.get(o, "other"), "spans": ivs}
                                for o, ivs in views.residency_spans(planned, log).items()]
        if "stalls" in want:
            out["stalls"] = views.stall_rows(planned, log)
        if "references" in want:
            out["references"] = views.reference_rows(planned)
        if "candidates" in want:
            out["candidates"] = views.candidate_rows(result) if result is not None else None
        return out

    @app.post("/api/compare")
    def compare_route(req: CompareRequest):
        import time
        hw = _hardware(req)
        prog = _program(req)
        names = req.policies or sorted(get_all_policies())
        lower = preview_workload(prog, hw)["compute_only_us"]
        rows = []
        for name in names:
            t0 = time.perf_counter()
            try:
                planned, _ = _plan(req, name, _cap(req.fast_memory_gib), prog, hw)
                log = simulate(planned)
                s = compute_summary(planned, log, prog, hw)
                rows.append({"policy": name, "ok": True, "makespan_us": s["makespan_us"], "tokens_per_s": s["tokens_per_s"],
                             "x_lower_bound": s["makespan_us"] / lower if lower else None, "peak_fast_bytes": s["peak_fast_bytes"],
                             "from_slow_bytes": s["from_slow_bytes"], "to_slow_bytes": s["to_slow_bytes"], "idle_pct": s["idle_pct"],
                             "planning_s": time.perf_counter() - t0})
            except HTTPException:
                raise
            except Exception as e:
                rows.append({"policy": name, "ok": False, "error": f"{type(e).__name__}: {str(e)[:300]}", "planning_s": time.perf_counter() - t0})
        good = [r for r in rows if r["ok"]]
        best = min(good, key=lambda r: r["makespan_us"])["policy"] if good else None
        return {"rows": rows, "best": best, "compute_only_us": lower}

    @app.post("/api/sweep")
    def sweep_route(req: SweepRequest):
        hw = _hardware(req)
        prog = _program(req)
        if not req.budgets_gib:
            raise HTTPException(status_code=422, detail="give `budgets_gib`")
        rows = []
        for gib in req.budgets_gib:
            try:
                planned, _ = _plan(req, req.policy, _cap(gib), prog, hw)
                s = compute_summary(planned, simulate(planned), prog, hw)
                rows.append({"budget_gib": gib, "ok": True, "makespan_us": s["makespan_us"], "tokens_per_s": s["tokens_per_s"],
                             "peak_fast_bytes": s["peak_fast_bytes"], "idle_pct": s["idle_pct"], "recompute_pct": s["recompute_pct"],
                             "from_slow_util_pct": s["from_slow_util_pct"], "to_slow_util_pct": s["to_slow_util_pct"]})
            except HTTPException:
                raise
            except Exception as e:
                rows.append({"budget_gib": gib, "ok": False, "error": f"{type(e).__name__}: {str(e)[:300]}"})
        return {"rows": rows, "policy": req.policy}

    @app.post("/api/validate")
    def validate_route(req: ValidateRequest):
        from ..schema import TaskChain
        from ..validate import RULES, STAGES
        try:
            chain = TaskChain.from_dict(req.chain)
        except (KeyError, TypeError, ValueError) as e:
            raise HTTPException(status_code=422, detail=f"not a task chain: {type(e).__name__}: {e}") from e
        stages = ("ids", "capacity") if req.planning_input else ("ids", "transfers", "lifetimes", "capacity")
        report = []
        ok = True
        for name in stages:
            if not ok:
                report.append({"stage": name, "ran": False, "problems": []})      # later stages assume the earlier ones passed
                continue
            found = STAGES[name](chain)
            ok = not found
            report.append({"stage": name, "ran": True,
                           "problems": [{"rule": p.rule, "meaning": RULES.get(p.rule, ""), "task": p.task, "object": p.obj, "text": str(p)}
                                        for p in found]})
        return {"valid": ok, "stages": report, "tasks": len(chain.tasks), "objects": len(chain.sizes())}

    return app


app = create_app()
