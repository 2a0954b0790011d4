"""Scaling fits over measured (n_gpus, tokens/s) points: efficiency against linear weak scaling, and a
least-squares fit of ``t(n) = t_compute + t_comm * (n - 1) / n`` (ring-style exposed communication) that
separates the exposed communication per step from the single-GPU step time.
Parity: reference ``src/dataflow_training/run/scaling.py:60``.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class ScalingFit:
    points: list[tuple[int, float]]             # (n, whole-job tokens/s)
    efficiency: dict[int, float]                # vs n x the single-GPU rate
    t_compute_ms: float
    t_comm_ms: float                            # exposed communication per step at large n
    residual: float


def fit_scaling(points: list[tuple[int, float]], tokens_per_gpu_step: float) -> ScalingFit:
    pts = sorted((int(n), float(v)) for n, v in points)
    base = next((v / n for n, v in pts if n == 1), pts[0][1] / pts[0][0])
    eff = {n: v / (n * base) for n, v in pts}
    # step time per point (weak scaling: per-GPU work fixed)
    xs = [(n - 1) / n for n, _ in pts]
    ys = [tokens_per_gpu_step * n / v * 1e3 for n, v in pts]
    m = len(pts)
    sx, sy = sum(xs), sum(ys)
    sxx, sxy = sum(x * x for x in xs), sum(x * y for x, y in zip(xs, ys))
    den = m * sxx - sx * sx
    if m < 2 or abs(den) < 1e-12:
        a, b = (ys[0] if ys else 0.0), 0.0
    else:
        b = (m * sxy - sx * sy) / den
        a = (sy - b * sx) / m
    res = sum((a + b * x - y) ** 2 for x, y in zip(xs, ys)) ** 0.5
    return ScalingFit(pts, eff, a, b, res)
