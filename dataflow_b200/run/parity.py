"""Curve comparison: is an engine loss curve inside a band around a reference curve, and is a curve healthy.
``Band`` is a relative tolerance that may widen with the step (bf16 trajectories diverge slowly).
Parity: reference ``src/dataflow_training/run/parity.py:16-120``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field


@dataclass(frozen=True)
class Band:
    rel: float = 3e-2              # tolerance at step 1
    growth: float = 0.0            # added per step
    abs_floor: float = 1e-6

    def tol(self, step: int, ref: float) -> float:
        return max((self.rel + self.growth * (step - 1)) * abs(ref), self.abs_floor)

    @staticmethod
    def named(name: str) -> "Band":
        return {"bitwise": Band(0.0, 0.0, 0.0), "fp32": Band(2e-4), "bf16": Band(3e-2, 5e-4), "loose": Band(1e-1, 1e-3)}[name]


@dataclass
class Comparison:
    ok: bool
    worst_step: int
    worst_rel: float
    mismatches: list[tuple[int, float, float]] = field(default_factory=list)

    def __bool__(self) -> bool:
        return self.ok


def compare(curve, reference, band: Band = Band()) -> Comparison:
    worst, worst_step, bad = 0.0, 0, []
    for i, (a, b) in enumerate(zip(curve, reference), 1):
        if not (math.isfinite(a) and math.isfinite(b)):
            bad.append((i, a, b))
            continue
        rel = abs(a - b) / max(abs(b), 1e-30)
        if rel > worst:
            worst, worst_step = rel, i
        if abs(a - b) > band.tol(i, b):
            bad.append((i, a, b))
    if len(curve) != len(reference):
        bad.append((min(len(curve), len(reference)) + 1, float("nan"), float("nan")))
    return Comparison(not bad, worst_step, worst, bad)


def curves_healthy(curve, *, must_decrease: bool = True, max_jump: float = 0.5) -> bool:
    """Finite everywhere, no single-step jump above ``max_jump`` (relative), and lower at the end than at the start."""
    if not curve or not all(math.isfinite(x) for x in curve):
        return False
    for a, b in zip(curve, curve[1:]):
        if b - a > max_jump * abs(a):
            return False
    return (curve[-1] < curve[0]) if must_decrease and len(curve) > 1 else True
