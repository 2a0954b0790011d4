"""Per-step trace summaries: time by compute key, lane busy time, compute-lane gaps.
Built from the always-on interval trace of a run (role of the reference's
``tools/bench/gap_census.py`` and the ``[plan]`` / step log lines)."""
from __future__ import annotations

from typing import Any


def summarize_trace(program, result) -> dict[str, Any]:
    by_id = {t.id: t for t in program.tasks}
    comp = sorted(result.trace.by_track("compute"), key=lambda i: i.start_us)
    keys: dict[str, list[float]] = {}
    for iv in comp:
        t = by_id.get(iv.name)
        k = (t.compute_block_key if t is not None else "?") or "?"
        if t is not None and any(m.startswith("dW") for m in t.mutates):
            k += "+acc"
        keys.setdefault(k, []).append(iv.end_us - iv.start_us)
    gaps = [b.start_us - a.end_us for a, b in zip(comp[:-1], comp[1:])]
    big = sorted(((b.start_us - a.end_us, b.name) for a, b in zip(comp[:-1], comp[1:])), reverse=True)[:8]
    out = {
        "makespan_ms": result.makespan_us / 1e3,
        "compute_busy_ms": sum(i.end_us - i.start_us for i in comp) / 1e3,
        "gap_total_ms": sum(g for g in gaps if g > 0) / 1e3,
        "gap_median_us": sorted(gaps)[len(gaps) // 2] if gaps else 0.0,
        "largest_gaps_ms": [(round(g / 1e3, 2), n) for g, n in big],
        "h2d_busy_ms": result.trace.busy_us("from_slow") / 1e3,
        "d2h_busy_ms": result.trace.busy_us("to_slow") / 1e3,
        "h2d_gbs": result.stats["h2d_bytes"] / max(result.trace.busy_us("from_slow"), 1e-9) / 1e3,
        "d2h_gbs": result.stats["d2h_bytes"] / max(result.trace.busy_us("to_slow"), 1e-9) / 1e3,
        "by_key_ms": {k: {"n": len(v), "total": round(sum(v) / 1e3, 2), "median": round(sorted(v)[len(v) // 2] / 1e3, 3)}
                      for k, v in sorted(keys.items())},
        "dispatch_ms": result.stats["dispatch_us_total"] / 1e3,
        "peak_fast_gib": result.peak_fast_bytes / 2 ** 30,
        "slab_overflows": result.slab_overflows,
    }
    return out
