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



def concurrent_pcie_probe(device: int, mib: int = 256, repeats: int = 16) -> tuple[float, float]:
    """(host-to-device, device-to-host) GB/s of this GPU with both directions busy; meant to be called by every rank of a
    node at the same moment (after a barrier), so that the figures are what the ranks get from the host TOGETHER."""
    from ..runtime import CudaBackend
    got = CudaBackend(device, "poll").measure_pcie(int(mib) << 20, int(repeats))
    return float(got["h2d_bidi_gbs"]), float(got["d2h_bidi_gbs"])


def hardware_as_shared(hw, world: int, device: int | None, probe=None):
    """The hardware row one of ``world`` ranks of a node should plan with.  The preset's share rule (``hw.shared``) is a guess
    at what the host delivers to several GPUs at once; how a box's GPUs hang off its sockets and switches decides the real
    figure (measured on this pool's 8 x B200 boxes with all ranks copying both ways: 45 GB/s per GPU at 2 ranks, 10-15 at
    8), and a plan priced with a rate the box does not deliver stalls on its prefetches.  So on devices every rank measures
    its host link while all the others do the same, the minimum over ranks (times 0.95) caps the row, and every rank plans
    with the same row.  ``DATAFLOW_PCIE_PROBE=0`` keeps the preset's guess."""
    import dataclasses
    import os
    shared = hw.shared(world)
    if world <= 1 or device is None or os.environ.get("DATAFLOW_PCIE_PROBE", "1") == "0":
        return shared
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return shared
    dist.barrier()
    try:
        h2d, d2h = (probe or concurrent_pcie_probe)(device)
    except Exception:       # noqa: BLE001  (a rank whose probe fails still joins the reduction below: zero = "keep the preset")
        h2d, d2h = 0.0, 0.0
    t = torch.tensor([h2d, d2h], dtype=torch.float64, device=torch.device("cuda", device) if torch.cuda.is_available() else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    h2d, d2h = (float(x) for x in t.tolist())
    if not (h2d > 0 and d2h > 0):
        return shared
    return dataclasses.replace(shared, h2d_gbs=min(hw.h2d_gbs, 0.95 * h2d), d2h_gbs=min(hw.d2h_gbs, 0.95 * d2h),
                               link_gbs=shared.link_gbs or hw.h2d_gbs)
