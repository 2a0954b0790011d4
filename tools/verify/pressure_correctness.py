"""Math invariance under memory pressure: the full annotated program of a preset through the REAL engine at descending
budgets.  The loss curve and every final weight must not depend on the budget (offloads, prefetches, evictions and
recompute move or rebuild bytes; they never change them): per-tensor relative L2 against the unconstrained run stays
at zero on the host backend and within bf16 noise on a device.

    python tools/verify/pressure_correctness.py --preset llama3:tiny --device cpu --budgets 0.06,0.04,0.03

Reference role: ``tools/verify/pressure_correctness.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from _cli import table  # noqa: E402


def run_at(fam, cfg, budget, device, steps):
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    tr = Trainer(fam, cfg, budget_gib=budget, device=device, hyper={"lr": 2e-3, "weight_decay": 0.1}, seed=3, leeway_bytes=0)
    try:
        losses = [tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, 64, 11, s)) for s in range(steps)]
        tr.sync_to_host()
        weights = {k: v.clone().float() for k, v in resolve_family(fam).bridge(cfg, tr.views_of).items()}
        info = {"recompute": sum(1 for v in tr.planned.recompute_levels.values() if v), "peak_gib": tr.last_result.peak_fast_bytes / 2 ** 30,
                "policy": tr.planned.policy}
    finally:
        tr.close()
    return losses, weights, info


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="llama3:tiny")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--budgets", default="0.06,0.04,0.03", help="GiB, descending")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    from dataflow_b200.run.presets import resolve_preset
    fam, cfg = resolve_preset(a.preset)
    device = None if a.device == "cpu" else int(a.device)
    tol = 1e-6 if device is None else 2e-2
    gold_l, gold_w, _ = run_at(fam, cfg, None, device, a.steps)
    rows, bad = [], 0
    for b in [float(x) for x in a.budgets.split(",")]:
        try:
            l, w, info = run_at(fam, cfg, b, device, a.steps)
        except Exception as e:
            rows.append({"budget": b, "note": f"no plan ({type(e).__name__})"})
            continue
        dl = max(abs(x - y) / abs(y) for x, y in zip(l, gold_l))
        dw = max(float((w[k] - gold_w[k]).norm() / (gold_w[k].norm() + 1e-30)) for k in gold_w)
        ok = dl <= tol and dw <= tol
        bad += not ok
        rows.append({"budget": b, "loss_rel": dl, "weight_rel_l2": dw, "recompute_layers": info["recompute"], "peak_gib": info["peak_gib"],
                     "policy": info["policy"], "note": "ok" if ok else "DIVERGED"})
    print(table(rows, [("budget", "{:.3f}"), ("loss_rel", "{:.2e}"), ("weight_rel_l2", "{:.2e}"), ("recompute_layers", "{}"),
                       ("peak_gib", "{:.4f}"), ("policy", "{}"), ("note", "{}")]))
    if a.out:
        json.dump(rows, open(a.out, "w"), indent=1)
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
