"""Ladder-3 sweep: every family x {uniform, ragged} through the model-step gate (engine versus twin from identical
weights and data), one table.

    python tools/verify/sweep_ladder3.py [--families llama3,olmoe] [--top 5]

Reference role: ``tools/verify/sweep_ladder3.py``.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from _cli import table  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--families", default=None)
    ap.add_argument("--top", type=int, default=3, help="worst tensors listed per cell")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--tol", type=float, default=1e-3)
    a = ap.parse_args(argv)
    from dataflow_b200.models.families import all_families
    from dataflow_b200.testing.family_gate import run_pair
    device = None if a.device == "cpu" else int(a.device)
    names = a.families.split(",") if a.families else sorted(n for n, f in all_families().items() if "tiny" in f.presets and f.twin)
    rows, bad = [], 0
    for fam in names:
        for shape in ("uniform", "ragged"):
            try:
                r = run_pair(fam, device=device, policy="fp32" if device is None else "bf16_master", shape=shape)
            except Exception as e:
                rows.append({"family": fam, "shape": shape, "note": f"ERROR {type(e).__name__}: {str(e)[:60]}"})
                bad += 1
                continue
            worst = sorted(r["weight_rel_l2"].items(), key=lambda kv: -kv[1])[:a.top]
            ok = r["max_loss_rel"] < (a.tol if device is None else 3e-2)
            bad += not ok
            rows.append({"family": fam, "shape": shape, "loss_rel": r["max_loss_rel"], "first": r["engine"][0], "last": r["engine"][-1],
                         "worst_tensors": ", ".join(f"{k}={v:.1e}" for k, v in worst), "note": "ok" if ok else "FAIL"})
    print(table(rows, [("family", "{}"), ("shape", "{}"), ("loss_rel", "{:.2e}"), ("first", "{:.4f}"), ("last", "{:.4f}"), ("note", "{}"),
                       ("worst_tensors", "{}")]))
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
