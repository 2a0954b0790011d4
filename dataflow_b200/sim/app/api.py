"""HTTP API of the simulator: presets, plan-free previews, and planned + simulated steps.

    GET  /api/health               liveness + version
    GET  /api/presets              hardware rows, model library, policies
    POST /api/workloads/preview    model (by name or explicit program) + training config + hardware -> totals, no plan
    POST /api/simulate             same input + memory budget + policy -> plan, simulate, summary, timelines

Reference role: ``src/dataflow_sim/app/server/main.py:78-211`` (request models), ``:216,221,346,552`` (the four routes).
``GET /`` serves a single-page front end (``static/index.html``: inputs, summary, compute / copy timeline, device-memory
curve, time by phase, work by phase, planner comparison, budget sweep, measured-run overlay from a trace file — plain JavaScript and SVG
over the four routes; the reference's is a React app).
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


def _hardware(req: WorkloadRequest) -> HardwareSpec:
    try:
        hw = get_hardware(req.hardware)
    except KeyError as e:
        raise HTTPException(status_code=404, detail=str(e)) from e
    if req.hardware_overrides:
        from dataclasses import replace
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

    @app.post("/api/simulate")
    def simulate_route(req: SimulateRequest):
        hw = _hardware(req)
        prog = _program(req)
        policies = get_all_policies()
        if req.policy not in policies:
            raise HTTPException(status_code=404, detail=f"unknown policy {req.policy!r}; known: {sorted(policies)}")
        cap = int(req.fast_memory_gib * (1 << 30)) if req.fast_memory_gib is not None else None
        try:
            chain = realize_workload(prog, hw, cap)
            planned = policies[req.policy](chain, chain.fast_memory_capacity, **req.policy_args)
            log = simulate(planned, memory_trace=req.memory_trace)
        except Exception as e:                      # planner / simulator refusals are the caller's answer, not a crash
            raise HTTPException(status_code=422, detail=f"{type(e).__name__}: {e}") from e
        out: dict[str, Any] = {"summary": compute_summary(planned, log, prog, hw), "preview": preview_workload(prog, hw),
                               "policy": req.policy, "metadata": prog.metadata}
        if req.timeline:
            out["timeline"] = [{"id": iv.task_id, "track": iv.track, "start": iv.start, "end": iv.end} for iv in log.task_intervals]
        if req.memory_trace:
            out["memory_trace"] = [{"t": p.t, "fast_bytes": p.fast_bytes, "workspace_bytes": p.workspace_bytes} for p in log.memory_trace]
        return out

    return app


app = create_app()
