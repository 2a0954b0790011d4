"""Planner registry: name → callable(chain, fast_memory_capacity, **kw) → annotated chain."""
from .pressurefit import (PREFETCH_RULES, RESIDENCY_SPECS, PlanningError, PressureFitResult,
                          apply_pressurefit_policy, pressurefit)


def get_all_policies():
    from . import baselines
    from .lookahead import apply_lookahead_policy
    return {
        "pressurefit": apply_pressurefit_policy,
        "lookahead": apply_lookahead_policy,
        "sliding_window": baselines.sliding_window,
        "belady_reactive": baselines.belady_reactive,
        "roundtrip": baselines.roundtrip_planner,
        "max_reduce": baselines.max_reduce,
        "min_grow": baselines.min_grow,
        "all_resident": baselines.all_resident,
    }
