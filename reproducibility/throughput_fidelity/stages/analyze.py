"""From measured cells to a verdict on the simulator: how far is measured from predicted, where, and why.

    overall      geometric mean, median, 10th / 90th percentile and worst of measured / predicted; share of cells within
                 5 % and within 10 %
    by axis      the same geometric mean per optimizer, sequence length, tokens per round and budget third (low / mid / high)
    by regime    cells split by what the plan is bound by: link-bound (a copy lane busy > 70 % of the predicted step),
                 recompute-heavy (> 15 % of the compute is recompute), compute-bound (the rest)
    causes       for the cells off by more than 10 %, what the measurement itself says: time lost between tasks when the plan
                 is replayed with the measured task durations (scheduling loss: the simulator's lane model is off) against the
                 rest (mis-priced tasks: the cost table is off); allocator overflows; a throttled device
"""
from __future__ import annotations

import math

from .common import geomean, quantile


def regime(pred_row: dict) -> str:
    if pred_row.get("link_pct", 0.0) > 70.0:
        return "link-bound"
    if pred_row.get("recomp_pct", 0.0) > 15.0:
        return "recompute-heavy"
    return "compute-bound"


def analyze(pred: list[dict], meas: list[dict]) -> dict:
    good = [m for m in meas if "ratio" in m]
    failed = [m for m in meas if "error" in m]
    if not good:
        return {"cells": 0, "failed": len(failed), "errors": [m["error"] for m in failed][:8]}
    ratios = [m["ratio"] for m in good]
    out = {"cells": len(good), "failed": len(failed), "geomean_ratio": geomean(ratios), "median_ratio": quantile(ratios, 0.5),
           "p10_ratio": quantile(ratios, 0.1), "p90_ratio": quantile(ratios, 0.9),
           "within_5pct": sum(abs(r - 1) <= 0.05 for r in ratios) / len(ratios),
           "within_10pct": sum(abs(r - 1) <= 0.10 for r in ratios) / len(ratios)}
    worst = max(good, key=lambda m: abs(math.log(m["ratio"])))
    out["worst"] = {k: worst.get(k) for k in ("cell", "opt", "seq", "t_round", "rounds", "budget", "ratio", "pred_s", "meas_s")}
    budgets = sorted(m["budget"] for m in good if m.get("budget") is not None)
    lo_cut, hi_cut = (quantile(budgets, 1 / 3), quantile(budgets, 2 / 3)) if budgets else (0.0, 0.0)

    def third(m):
        b = m.get("budget")
        return "unbounded" if b is None else ("low" if b <= lo_cut else "high" if b > hi_cut else "mid")

    axes = {"opt": lambda m: m.get("opt"), "seq": lambda m: m.get("seq"), "t_round": lambda m: m.get("t_round"), "budget_third": third,
            "regime": lambda m: regime(pred[m["cell"]]) if m.get("cell") is not None and m["cell"] < len(pred) else "?"}
    out["by_axis"] = {}
    for name, key in axes.items():
        groups: dict = {}
        for m in good:
            groups.setdefault(str(key(m)), []).append(m["ratio"])
        out["by_axis"][name] = {k: {"cells": len(v), "geomean_ratio": geomean(v), "worst": max(v, key=lambda r: abs(math.log(r)))}
                                for k, v in sorted(groups.items())}
    off = []
    for m in good:
        if abs(m["ratio"] - 1) <= 0.10:
            continue
        gap = m.get("replay_gap_pct")
        why = []
        if gap is not None:
            # measured = replay of the plan with measured task times + gap: the gap is scheduling the simulator did not see
            excess = 100.0 * (m["ratio"] - 1)
            why.append(f"scheduling loss {gap:.1f} % of the step, task pricing {excess - gap:+.1f} %")
        if m.get("overflows"):
            why.append(f"{m['overflows']} allocator overflows")
        reasons = (m.get("clocks") or {}).get("reasons") or []
        if any(r != "sw_power_cap" for r in reasons):
            why.append("device throttled: " + ", ".join(reasons))
        off.append({"cell": m.get("cell"), "ratio": m["ratio"], "budget": m.get("budget"), "why": "; ".join(why) or "unexplained"})
    out["off_by_more_than_10pct"] = off
    return out
