#!/usr/bin/env python
"""Which tasks does the cost table mis-price?  Runs a preset for a few steps, takes the measured duration of every task from
the last step's trace, and sets it against the duration the plan was made with.  Tasks are grouped by kind (the task id
without its round and layer numbers); per kind: calls, predicted and measured time, their ratio, and the share of the
step's total mis-pricing the kind is responsible for.  The kinds at the top are where a better cost (a measured profile, a
fixed roofline term) pays.

    python reproducibility/throughput_fidelity/diagnostics/task_cost_audit.py --preset llama3_8b --budget 60 --device 0
    python reproducibility/throughput_fidelity/diagnostics/task_cost_audit.py --preset llama3:tiny --device cpu
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, ROOT)


def kind_of(task_id: str) -> str:
    return re.sub(r"(_\d+)+$", "", task_id)


def audit(program, trace) -> dict:
    from dataflow_b200.lowering.replay import measured_durations
    meas = measured_durations(trace)
    kinds: dict[str, dict] = {}
    for t in program.tasks:
        if t.id not in meas:
            continue
        k = kinds.setdefault(kind_of(t.id), {"calls": 0, "pred_us": 0.0, "meas_us": 0.0})
        k["calls"] += 1
        k["pred_us"] += float(t.runtime_us)
        k["meas_us"] += float(meas[t.id])
    total_err = sum(abs(k["meas_us"] - k["pred_us"]) for k in kinds.values()) or 1.0
    rows = []
    for name, k in kinds.items():
        rows.append({"kind": name, **k, "ratio": k["meas_us"] / k["pred_us"] if k["pred_us"] else float("inf"),
                     "share_of_mispricing_pct": 100.0 * abs(k["meas_us"] - k["pred_us"]) / total_err})
    rows.sort(key=lambda r: -r["share_of_mispricing_pct"])
    pred, got = sum(r["pred_us"] for r in rows), sum(r["meas_us"] for r in rows)
    return {"tasks": sum(r["calls"] for r in rows), "pred_compute_us": pred, "meas_compute_us": got, "ratio": got / pred if pred else float("inf"),
            "kinds": rows}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="llama3:tiny")
    ap.add_argument("--budget", type=float, default=None)
    ap.add_argument("--device", default="0")
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--profile", action="store_true", help="plan with per-task costs measured on the device first")
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    from dataflow_b200.run.presets import resolve_preset
    fam, cfg = resolve_preset(a.preset)
    device = None if a.device == "cpu" else int(a.device)
    tr = Trainer(fam, cfg, budget_gib=a.budget, device=device, profile=a.profile and device is not None)
    try:
        vocab = getattr(cfg, "vocab_size", 1024)
        for s in range(max(a.steps, 2)):
            tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, vocab, 0, s, pin=device is not None))
        res = audit(tr.program, tr.last_result.trace)
    finally:
        tr.close()
    print(f"{res['tasks']} tasks: compute predicted {res['pred_compute_us'] / 1e3:.2f} ms, measured {res['meas_compute_us'] / 1e3:.2f} ms "
          f"(ratio {res['ratio']:.3f})")
    print(f"{'kind':<28}{'calls':>6}{'pred ms':>11}{'meas ms':>11}{'ratio':>8}{'share %':>9}")
    for r in res["kinds"][:14]:
        print(f"{r['kind']:<28}{r['calls']:>6}{r['pred_us'] / 1e3:>11.3f}{r['meas_us'] / 1e3:>11.3f}{r['ratio']:>8.2f}{r['share_of_mispricing_pct']:>9.1f}")
    if a.json:
        with open(a.json, "w") as f:
            json.dump(res, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
