"""Recompute selection on top of PressureFit.

Each saved-context object may carry recompute options (``RecomputeRewrite``): level 0
keeps the full context, higher levels keep less and add a recompute task in front of
the backward.  The selector prices whole assignments by re-lowering
(``build_variant(levels)``), planning and simulating them: seeds *none*, *all* and
*every other layer*, then an evidence-directed greedy pass that flips the layers
whose context the best plan so far had to stream through backing memory.  Role
parity: reference ``src/dataflow_sim/planning/recompute.py:48-224``.
"""
from __future__ import annotations

import re
from typing import Callable, Mapping

from ..policies.pressurefit import PlanningError


def _layers_with_rewrites(program) -> list[int]:
    out = set()
    for rw in program.recompute_rewrites:
        m = re.match(r"layer(\d+)", rw.group_key or "")
        if m:
            out.add(int(m.group(1)))
    return sorted(out)


def _streamed_context_layers(planned) -> list[int]:
    hit: dict[int, int] = {}
    for t in planned.program.tasks:
        for d in t.offload_after:
            m = re.match(r"A_\d+_\d+_(\d+)$", d.object_id)
            if m:
                hit[int(m.group(1))] = hit.get(int(m.group(1)), 0) + 1
    return [k for k, _ in sorted(hit.items(), key=lambda kv: -kv[1])]


def plan_with_recompute(program, fast_memory_capacity, build_variant: Callable[[Mapping[int, int]], object], *,
                        backing_memory_capacity=None, leeway_bytes=None, max_evals: int = 8, level: int = 1):
    from ...lowering.planning import DEFAULT_PROGRAM_LEEWAY_BYTES, plan_program
    leeway = DEFAULT_PROGRAM_LEEWAY_BYTES if leeway_bytes is None else leeway_bytes
    layers = _layers_with_rewrites(program)
    tried: dict[tuple, object] = {}

    def price(levels: Mapping[int, int]):
        key = tuple(sorted((k, v) for k, v in levels.items() if v))
        if key in tried:
            return tried[key]
        prog = program if not key else build_variant(dict(key))
        try:
            p = plan_program(prog, fast_memory_capacity, recompute=False,
                             backing_memory_capacity=backing_memory_capacity, leeway_bytes=leeway)
            p.recompute_levels = dict(key)
        except PlanningError:
            p = None
        tried[key] = p
        return p

    best = price({})
    if best is not None and best.makespan_us <= best.lower_bound_us * (1 + 1e-6):
        return best                                        # nothing to gain: the plan is compute-bound already
    seeds = [{l: level for l in layers}, {l: level for l in layers[::2]}]
    for s in seeds:
        c = price(s)
        if c is not None and (best is None or c.makespan_us < best.makespan_us):
            best = c
    if best is None:
        raise PlanningError("no recompute assignment fits the budget")
    evals = len(tried)
    improved = True
    while improved and evals < max_evals:
        improved = False
        cur = dict(best.recompute_levels)
        streamed = [l for l in _streamed_context_layers(best) if not cur.get(l)]
        for l in streamed[:2]:
            trial = dict(cur)
            trial[l] = level
            c = price(trial)
            evals += 1
            if c is not None and c.makespan_us < best.makespan_us * (1 - 1e-4):
                best, improved = c, True
                break
            if evals >= max_evals:
                break
    return best
