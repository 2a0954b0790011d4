"""Summarise one or more training runs from their result files (``train.py ... --out run.json``): final and best loss,
tokens/s (median of the steady steps), step-time percentiles, and a coarse text plot of the curve.

    python tools/train/pretrain_report.py run_a.json run_b.json

Reference role: ``tools/train/pretrain_report.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from _cli import table  # noqa: E402


def spark(values, width=48):
    if not values:
        return ""
    bars = " .:-=+*#%@"
    step = max(len(values) // width, 1)
    pts = [sum(values[i:i + step]) / len(values[i:i + step]) for i in range(0, len(values), step)]
    lo, hi = min(pts), max(pts)
    return "".join(bars[int((v - lo) / (hi - lo + 1e-12) * (len(bars) - 1))] for v in pts)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("runs", nargs="+")
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args(argv)
    rows = []
    for path in a.runs:
        d = json.load(open(path))
        losses = d.get("losses") or d.get("curve") or []
        times = d.get("step_wall_s") or d.get("step_s") or []
        steady = sorted(times[a.warmup:]) or sorted(times)
        tok = d.get("tokens_per_step") or 0
        rows.append({"run": os.path.basename(path), "steps": len(losses), "first": losses[0] if losses else None,
                     "final": losses[-1] if losses else None, "best": min(losses) if losses else None,
                     "s_step_p50": steady[len(steady) // 2] if steady else None, "s_step_p90": steady[int(len(steady) * 0.9)] if steady else None,
                     "tok_s": tok / steady[len(steady) // 2] if steady and tok else None, "curve": spark(losses)})
    print(table(rows, [("run", "{}"), ("steps", "{}"), ("first", "{:.4f}"), ("final", "{:.4f}"), ("best", "{:.4f}"), ("s_step_p50", "{:.4f}"),
                       ("s_step_p90", "{:.4f}"), ("tok_s", "{:.0f}"), ("curve", "{}")]))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
