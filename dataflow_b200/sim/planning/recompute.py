"""Recompute selection on top of PressureFit.

Each saved-context object may carry recompute options (``RecomputeRewrite``): level 0
keeps the full context, higher levels keep less and add a recompute task in front of
the backward.  The selector prices whole assignments by re-lowering
(``build_variant(levels)``), planning and simulating them:

* seeds: nothing recomputed, every layer at each offered level;
* a sweep over *how many* layers run at each level (evenly spread over depth);
* a local refinement that moves the count up or down while the makespan improves.

The search uses a reduced PressureFit portfolio; the winner is re-planned with the
full one.  Role parity: reference ``src/dataflow_sim/planning/recompute.py:48-224``.
"""
from __future__ import annotations

import re
from typing import Callable, Mapping

from ..policies.pressurefit import PREFETCH_RULES, RESIDENCY_SPECS, PlanningError


def _layers_and_levels(program) -> tuple[list[int], list[int]]:
    layers, levels = set(), set()
    for rw in program.recompute_rewrites:
        m = re.match(r"layer(\d+)", rw.group_key or "")
        if m:
            layers.add(int(m.group(1)))
        for o in rw.options:
            if o.level:
                levels.add(o.level)
    return sorted(layers), sorted(levels)


def spread(layers: list[int], k: int) -> list[int]:
    """``k`` layers evenly spread over ``layers``."""
    if k <= 0:
        return []
    if k >= len(layers):
        return list(layers)
    step = len(layers) / k
    return sorted({layers[min(int(i * step + step / 2), len(layers) - 1)] for i in range(k)})


def plan_with_recompute(program, fast_memory_capacity, build_variant: Callable[[Mapping[int, int]], object], *,
                        backing_memory_capacity=None, leeway_bytes=None, max_evals: int = 24):
    from ...lowering.planning import DEFAULT_PROGRAM_LEEWAY_BYTES, plan_program
    leeway = DEFAULT_PROGRAM_LEEWAY_BYTES if leeway_bytes is None else leeway_bytes
    layers, levels = _layers_and_levels(program)
    quick_specs = [s for s in RESIDENCY_SPECS if s.name in ("belady", "bytes_x_distance")]
    quick_rules = [r for r in PREFETCH_RULES if r.name in ("jit_1.0", "jit_1.6", "window_2")]
    tried: dict[tuple, object] = {}
    evals = 0

    def price(assign: Mapping[int, int], full: bool = False):
        nonlocal evals
        key = tuple(sorted(((k, v) for k, v in assign.items() if v), key=lambda kv: (str(type(kv[0])), kv)))
        if not full and key in tried:
            return tried[key]
        prog = program if not key else build_variant(dict(key))
        try:
            p = plan_program(prog, fast_memory_capacity, recompute=False,
                             backing_memory_capacity=backing_memory_capacity, leeway_bytes=leeway,
                             specs=None if full else quick_specs, rules=None if full else quick_rules,
                             quick=not full)
            p.recompute_levels = dict(key)
        except PlanningError:
            p = None
        if not full:
            tried[key] = p
            evals += 1
        return p

    def better(a, b):
        return a is not None and (b is None or a.makespan_us < b.makespan_us * (1 - 1e-5))

    best = price({})
    if best is not None and best.makespan_us <= best.lower_bound_us * (1 + 1e-6):
        return price({}, full=True) or best
    L = len(layers)
    R = int((program.metadata or {}).get("grad_accum_rounds", 1))
    # (a) recompute only in the last round(s): their backward is where optimizer state streams in, so freeing
    #     those rounds' activations buys room to prefetch the state ahead of the optimizer tasks, while the
    #     other rounds keep streaming activations over lanes that are otherwise idle
    best_tail: dict = {}
    if R > 1:
        tail_best = None
        for lv in reversed(levels):
            for nlast in (L, (3 * L) // 4, L // 2):
                if nlast <= 0:
                    continue
                trial = {(R - 1, l): lv for l in spread(layers, nlast)}
                c = price(trial)
                if better(c, tail_best):
                    tail_best, best_tail = c, trial
                if better(c, best):
                    best = c
        if R > 2 and best_tail:
            lv = next(iter(best_tail.values()))
            trial = dict(best_tail)
            trial.update({(R - 2, l): lv for l in spread(layers, L // 2)})
            c = price(trial)
            if better(c, best):
                best = c
    # (b) the same level in every round, for all layers and for spread subsets
    uniform_best, best_uniform = None, {}
    for lv in levels:
        for k in (L, (3 * L) // 4, L // 2, L // 4):
            if evals >= max_evals + 8 or k <= 0:
                continue
            trial = {l: lv for l in spread(layers, k)}
            c = price(trial)
            if better(c, uniform_best):
                uniform_best, best_uniform = c, trial
            if better(c, best):
                best = c
    # (c) both together
    if best_tail and best_uniform and evals < max_evals + 12:
        trial = dict(best_uniform)
        trial.update(best_tail)
        c = price(trial)
        if better(c, best):
            best = c
    if best is None:
        raise PlanningError("no recompute assignment fits the budget")
    # local refinement of the winning count
    cur = dict(best.recompute_levels)
    if cur and len(set(cur.values())) == 1 and all(isinstance(k, int) for k in cur):
        lv = next(iter(cur.values()))
        k = len(cur)
        step = max(L // 8, 1)
        while evals < max_evals and step >= 1:
            moved = False
            for nk in (k - step, k + step):
                if 0 < nk <= L and evals < max_evals:
                    c = price({l: lv for l in spread(layers, nk)})
                    if better(c, best):
                        best, k, moved = c, nk, True
                        break
            if not moved:
                step //= 2
    final = price(dict(best.recompute_levels), full=True)
    return final if better(final, best) or final is not None and final.makespan_us <= best.makespan_us else best
