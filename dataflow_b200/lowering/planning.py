"""Plan a bare Program against a fast-memory budget.

``budget = planned object pool + largest task workspace + leeway``: the planner is
given ``budget - leeway - max(workspace)`` for declared objects, so the executor's
slab (objects) plus the framework allocator's scratch (workspace) stay under the
budget on the device.  The directives come from the best of two planners, both verified
by the simulator: Lookahead (decides inside a simulation run) and PressureFit (offline
residency sweep), optionally wrapped by the recompute planner; the result is returned with its
predicted makespan, peaks and transfer statistics.  Role parity: reference
``src/dataflow_training/lowering/planning.py:22-356``.
"""
from __future__ import annotations

import os

from dataclasses import dataclass, field, replace
from typing import Any, Callable, Mapping

from ..core import Program, apply_chain_annotations, to_sim_chain
from ..sim import run as simulate
from ..sim.policies.pressurefit import PlanningError, pressurefit

DEFAULT_PROGRAM_LEEWAY_BYTES = int(1.5 * (1 << 30))


@dataclass
class PlannedProgram:
    program: Program
    makespan_us: float
    lower_bound_us: float
    peak_fast_bytes: int
    peak_backing_bytes: int
    object_capacity: int
    max_workspace: int
    budget: int | None
    policy: str
    recompute_levels: dict[int, int] = field(default_factory=dict)
    transfer: dict[str, Any] = field(default_factory=dict)
    candidates: int = 0

    @property
    def idle_fraction(self) -> float:
        return 0.0 if not self.makespan_us else 1.0 - self.lower_bound_us / self.makespan_us


def transfer_summary(log) -> dict[str, Any]:
    out: dict[str, Any] = {}
    for d in ("from_slow", "to_slow"):
        ivs = log.transfer_intervals(d)
        out[d] = {"count": len(ivs), "busy_us": sum(i.end - i.start for i in ivs)}
    out["makespan_us"] = log.makespan
    for d in ("from_slow", "to_slow"):
        out[d]["busy_fraction"] = out[d]["busy_us"] / log.makespan if log.makespan else 0.0
    return out


def strip_plan_annotations(program: Program) -> Program:
    return replace(program, tasks=tuple(t.with_directives(releases_after=(), offload_after=(), prefetch_after=())
                                        for t in program.tasks),
                   initial_objects=_dedup_initial(program), fast_memory_capacity=None)


def _dedup_initial(program: Program):
    seen, out = set(), []
    for o in program.initial_objects:
        if o.id in seen:
            continue
        seen.add(o.id)
        out.append(replace(o, location="backing") if o.persistent or o.role == "input" else o)
    return tuple(out)


def plan_program(program: Program, fast_memory_capacity: int | None, *, recompute: bool = False,
                 build_variant: Callable[[Mapping[int, int]], Program] | None = None,
                 backing_memory_capacity: int | None = None,
                 leeway_bytes: int = DEFAULT_PROGRAM_LEEWAY_BYTES, policy: str = "auto",
                 specs=None, rules=None, lookahead_specs=None, quick: bool = False) -> PlannedProgram:
    """``fast_memory_capacity`` is the whole device budget in bytes (``None`` = unbounded).

    ``policy``: ``"auto"`` (best of Lookahead and PressureFit), ``"wide"`` (``auto`` plus the span planners ``max_reduce``,
    ``min_grow`` and ``roundtrip``: on the planner corpus the best of the five is 1.8 % faster in the geometric mean
    than the best of the two, for about half as much planning time again), ``"lookahead"``, ``"pressurefit"`` or any name of
    ``sim.policies.get_all_policies()``.  ``DATAFLOW_PLANNER`` replaces ``auto`` by another policy for a whole run.
    ``quick`` keeps ``auto`` to a few Lookahead candidates (used by searches that price many program variants)."""
    levels: dict[int, int] = {}
    if policy == "auto":
        policy = os.environ.get("DATAFLOW_PLANNER", "auto")
    wide = policy == "wide"
    if wide:
        policy = "auto"
    if recompute and build_variant is not None and program.recompute_rewrites:
        from ..sim.planning.recompute import plan_with_recompute
        return plan_with_recompute(program, fast_memory_capacity, build_variant,
                                   backing_memory_capacity=backing_memory_capacity, leeway_bytes=leeway_bytes)
    max_ws = max((t.workspace_bytes for t in program.tasks), default=0)
    cap = None
    if fast_memory_capacity is not None:
        cap = int(fast_memory_capacity) - int(leeway_bytes) - max_ws
        if cap <= 0:
            raise PlanningError(f"budget {fast_memory_capacity} leaves no room after workspace {max_ws} and leeway {leeway_bytes}")
    chain = to_sim_chain(program, with_directives=False)
    chain = replace(chain, tasks=[replace(t, workspace_bytes=0) for t in chain.tasks],
                    backing_memory_capacity=backing_memory_capacity)
    if policy in ("auto", "lookahead", "pressurefit"):
        from ..sim.policies.lookahead import LOOKAHEAD_SPECS, lookahead
        best_chain, best_ms, ncand, errors = None, float("inf"), 0, []
        if policy != "pressurefit":
            la = lookahead_specs
            if la is None and quick:
                la = [x for x in LOOKAHEAD_SPECS if x.name in ("cost_aware", "cost_aware_wide", "bytes")]
            try:
                r = lookahead(chain, cap, specs=la, headrooms=(0.02,) if quick else (0.02, 0.05))
                best_chain, best_ms, ncand = r.chain, r.makespan, len(r.candidates)
                policy_used = f"lookahead:{r.chosen.spec}"
            except PlanningError as e:
                errors.append(str(e))
        lower = float(sum(t.runtime for t in chain.tasks))
        if policy == "pressurefit" or (policy == "auto" and not quick and best_ms > lower * (1 + 1e-9)) \
                or best_chain is None and policy == "auto":
            try:
                res = pressurefit(chain, cap, specs=specs, rules=rules)
                ncand += len(res.candidates)
                if res.makespan < best_ms:
                    best_chain, best_ms = res.chain, res.makespan
                    policy_used = f"pressurefit:{res.chosen.spec}/{res.chosen.rule}"
            except PlanningError as e:
                errors.append(str(e))
        if wide and not quick and (best_chain is None or best_ms > lower * (1 + 1e-9)):
            from ..sim.policies import get_all_policies
            table = get_all_policies()
            for name in ("max_reduce", "min_grow", "roundtrip"):
                try:
                    cand = table[name](chain, cap)
                    ms = simulate(cand, validate=False).makespan
                except (PlanningError, ValueError) as e:          # no plan of this shape, or a chain this planner refuses
                    errors.append(str(e))
                    continue
                ncand += 1
                if ms < best_ms:
                    best_chain, best_ms, policy_used = cand, ms, name
        if best_chain is None:
            raise PlanningError("; ".join(errors))
        planned_chain, policy = best_chain, policy_used
    else:
        from ..sim.policies import get_all_policies
        planned_chain, ncand = get_all_policies()[policy](chain, cap), 1
    log = simulate(planned_chain, validate=False)
    annotated = apply_chain_annotations(program, planned_chain)
    annotated = replace(annotated, metadata={**dict(annotated.metadata), "workspace_accounting": "external",
                                             "max_workspace_bytes": max_ws, "budget_bytes": fast_memory_capacity})
    return PlannedProgram(annotated, log.makespan, float(sum(t.runtime_us for t in program.tasks)),
                          log.peak_fast_memory_bytes, log.peak_backing_memory_bytes, cap if cap is not None else 0,
                          max_ws, fast_memory_capacity, policy, levels, transfer_summary(log), ncand)
