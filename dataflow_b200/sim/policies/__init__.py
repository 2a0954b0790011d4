"""Planner registry: name → callable(chain, fast_memory_capacity, **kw) → annotated chain."""
from .pressurefit import (PREFETCH_RULES, RESIDENCY_SPECS, PlanningError, PressureFitResult,
                          apply_pressurefit_policy, pressurefit)


def get_all_policies():
    from . import baselines, max_reduce, min_grow, reactive, roundtrip, sliding_window
    from .lookahead import apply_lookahead_policy
    return {
        "pressurefit": apply_pressurefit_policy,
        "lookahead": apply_lookahead_policy,
        "sliding_window": sliding_window.sliding_window,
        "belady_reactive": reactive.belady_reactive,
        "roundtrip": roundtrip.roundtrip_planner,
        "max_reduce": max_reduce.max_reduce,
        "min_grow": min_grow.min_grow,
        "all_resident": baselines.all_resident,
    }
