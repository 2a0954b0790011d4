"""Accuracy fidelity study: the loss curve of a preset must not depend on the device budget, and must track the pure-torch
twin trained from the same weights on the same data.

Stages (JSON per stage in ``--out``; ``--resume`` keeps finished ones):

    twin        the twin's curve (CPU fp32): the reference trajectory
    budgets     ``--auto-budgets`` picks three budgets from the plan: unconstrained, ~60% and ~35% of the all-resident peak
    engine      the engine's curve at every budget
    analyze     per budget: max relative distance to the twin and to the unconstrained engine run; ``report.md``

    python reproducibility/accuracy_fidelity/run_accuracy.py --preset llama3:tiny --device cpu --steps 8 --auto-budgets --out /tmp/acc

Reference role: ``reproducibility/accuracy_fidelity/run_accuracy.py``.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def stage(out, name, resume, fn):
    path = os.path.join(out, name + ".json")
    if resume and os.path.exists(path):
        print(f"[{name}] kept {path}")
        return json.load(open(path))
    t0 = time.time()
    val = fn()
    json.dump(val, open(path, "w"), indent=1)
    print(f"[{name}] done in {time.time() - t0:.1f}s")
    return val


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="llama3:tiny")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--ga-rounds", type=int, default=None)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--peak-lr", type=float, default=2e-3)
    ap.add_argument("--budgets", default=None, help="GiB list")
    ap.add_argument("--auto-budgets", action="store_true")
    ap.add_argument("--device", default="0")
    ap.add_argument("--policy", default=None, help="dtype policy (default: fp32 on cpu, bf16_master on a device)")
    ap.add_argument("--out", required=True)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--stages", default="twin,budgets,engine,analyze")
    a = ap.parse_args(argv)
    os.makedirs(a.out, exist_ok=True)
    device = None if a.device == "cpu" else int(a.device)
    from dataflow_b200.run.presets import resolve_preset
    from dataflow_b200.testing.family_gate import run_pair
    fam, cfg = resolve_preset(a.preset)
    preset = a.preset.split(":", 1)[1] if ":" in a.preset else a.preset
    over = {k: v for k, v in (("batch", a.batch), ("grad_accum_rounds", a.ga_rounds)) if v}
    policy = a.policy or ("fp32" if device is None else "bf16_master")
    hyper = {"lr": a.peak_lr, "weight_decay": 0.1}
    stages = a.stages.split(",")

    def pair(budget):
        return run_pair(fam, device=device, policy=policy, steps=a.steps, budget_gib=budget, hyper=hyper, preset=preset, overrides=over)

    base = stage(a.out, "twin", a.resume, lambda: pair(None)) if "twin" in stages else None

    def pick():
        if a.budgets:
            return [float(x) for x in a.budgets.split(",")]
        from dataflow_b200.run.driver import plan_at_budget
        full = plan_at_budget(fam, dataclasses.replace(cfg, dtype_policy=policy, **over), None).peak_fast_bytes / 2 ** 30
        return [round(full * 0.6, 4), round(full * 0.35, 4)]
    budgets = stage(a.out, "budgets", a.resume, pick) if "budgets" in stages else []

    def engine():
        runs = {}
        for b in budgets:
            try:
                runs[str(b)] = pair(b)["engine"]
            except Exception as e:
                runs[str(b)] = {"error": f"{type(e).__name__}: {e}"}
        return runs
    runs = stage(a.out, "engine", a.resume, engine) if "engine" in stages else {}
    if "analyze" in stages and base:
        rel = lambda x, y: max(abs(p - q) / abs(q) for p, q in zip(x, y))  # noqa: E731
        lines = ["# Accuracy fidelity", "", f"preset `{a.preset}`, {a.steps} steps, dtype policy `{policy}`", "",
                 "| budget GiB | max rel. distance to the twin | to the unconstrained engine run | final loss |", "|---|---|---|---|",
                 f"| unconstrained | {rel(base['engine'], base['twin']):.2e} | 0 | {base['engine'][-1]:.4f} |"]
        worst = 0.0
        for b, curve in runs.items():
            if isinstance(curve, dict):
                lines.append(f"| {b} | {curve['error']} | | |")
                continue
            d = rel(curve, base["engine"])
            worst = max(worst, d)
            lines.append(f"| {b} | {rel(curve, base['twin']):.2e} | {d:.2e} | {curve[-1]:.4f} |")
        open(os.path.join(a.out, "report.md"), "w").write("\n".join(lines) + "\n")
        print(f"[analyze] worst budget-to-budget distance {worst:.2e}; twin distance {rel(base['engine'], base['twin']):.2e}")
        return 0 if worst < (1e-5 if device is None else 3e-2) else 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
