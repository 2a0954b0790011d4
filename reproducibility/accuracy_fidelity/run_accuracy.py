"""Accuracy fidelity study: the loss curve of a preset must not depend on the device budget, and must track the pure-torch
twin trained from the same weights on the same data.

Stages (JSON per stage in ``--out``; ``--resume`` keeps finished ones):

    twin        the twin's curve (CPU fp32): the reference trajectory
    budgets     ``--auto-budgets`` picks three budgets from the plan: unconstrained, ~60% and ~35% of the all-resident peak
    engine      the engine's curve at every budget
    analyze     per budget: max and final relative distance to the twin and to the unconstrained engine run, the step at
                which the curves are farthest apart, the distance of the final weights from the twin's per tensor (worst
                tensors named); ``report.md``, ``curves.svg`` (every curve on one plot) and ``curves.json``

The run passes when the curves at every budget agree with the unconstrained engine run (a plan moves bytes, it must not
change numbers: 1e-5 in fp32 on the CPU backend, 3 % with bf16 kernels on a device) and the engine tracks the twin.

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
                r = pair(b)
                worst = sorted(r["weight_rel_l2"].items(), key=lambda kv: -kv[1])[:3]
                runs[str(b)] = {"curve": r["engine"], "max_weight_rel_l2": r["max_weight_rel_l2"], "worst_tensors": worst}
            except Exception as e:
                runs[str(b)] = {"error": f"{type(e).__name__}: {e}"}
        return runs
    runs = stage(a.out, "engine", a.resume, engine) if "engine" in stages else {}
    if "analyze" in stages and base:
        def rel(x, y):
            d = [abs(p - q) / abs(q) for p, q in zip(x, y)]
            return max(d), d[-1], d.index(max(d))
        t_max, t_last, t_at = rel(base["engine"], base["twin"])
        lines = ["# Accuracy fidelity", "", f"preset `{a.preset}`, {a.steps} steps, dtype policy `{policy}`, peak lr {a.peak_lr}", "",
                 "| budget GiB | max rel. distance to the twin (at step) | final | max to the unconstrained engine run | final loss | "
                 "final weights: max rel. L2 to the twin | worst tensors |", "|---|---|---|---|---|---|---|",
                 f"| unconstrained | {t_max:.2e} ({t_at}) | {t_last:.2e} | 0 | {base['engine'][-1]:.4f} | {base['max_weight_rel_l2']:.2e} | "
                 + ", ".join(f"{k} {v:.1e}" for k, v in sorted(base['weight_rel_l2'].items(), key=lambda kv: -kv[1])[:3]) + " |"]
        worst = 0.0
        curves = {"twin": base["twin"], "unconstrained": base["engine"]}
        for b, run in runs.items():
            if "error" in run:
                lines.append(f"| {b} | {run['error']} | | | | | |")
                continue
            curve = run["curve"]
            curves[f"{b} GiB"] = curve
            d, _, _ = rel(curve, base["engine"])
            m, last, at = rel(curve, base["twin"])
            worst = max(worst, d)
            lines.append(f"| {b} | {m:.2e} ({at}) | {last:.2e} | {d:.2e} | {curve[-1]:.4f} | {run['max_weight_rel_l2']:.2e} | "
                         + ", ".join(f"{k} {v:.1e}" for k, v in run["worst_tensors"]) + " |")
        with open(os.path.join(a.out, "report.md"), "w") as f:
            f.write("\n".join(lines) + "\n")
        with open(os.path.join(a.out, "curves.json"), "w") as f:
            json.dump(curves, f, indent=1)
        with open(os.path.join(a.out, "curves.svg"), "w") as f:
            f.write(curves_svg(curves))
        print(f"[analyze] worst budget-to-budget distance {worst:.2e}; twin distance {t_max:.2e}")
        return 0 if worst < (1e-5 if device is None else 3e-2) else 1
    return 0


def curves_svg(curves: dict) -> str:
    """Every loss curve on one plot, as stand-alone SVG text."""
    W, H, P = 640, 380, 50
    ys = [v for c in curves.values() for v in c]
    n = max(len(c) for c in curves.values())
    lo, hi = min(ys), max(ys)
    hi = hi if hi > lo else lo + 1.0
    sx = lambda i: P + i / max(n - 1, 1) * (W - P - 16)          # noqa: E731
    sy = lambda v: H - P - (v - lo) / (hi - lo) * (H - P - 24)   # noqa: E731
    colors = ["#1b1f24", "#4c8bf5", "#e5534b", "#57ab5a", "#d4a72c", "#986ee2"]
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" viewBox="0 0 {W} {H}" width="{W}" height="{H}" font-family="sans-serif" font-size="11">',
           f'<rect width="{W}" height="{H}" fill="#fff"/><line x1="{P}" y1="{H - P}" x2="{W - 16}" y2="{H - P}" stroke="#333"/>'
           f'<line x1="{P}" y1="{H - P}" x2="{P}" y2="24" stroke="#333"/><text x="{W / 2}" y="{H - 14}" text-anchor="middle">step</text>'
           f'<text x="{P - 6}" y="{sy(lo) + 4:.1f}" text-anchor="end">{lo:.3f}</text><text x="{P - 6}" y="{sy(hi) + 4:.1f}" text-anchor="end">{hi:.3f}</text>']
    for k, (name, c) in enumerate(curves.items()):
        col = colors[k % len(colors)]
        dash = ' stroke-dasharray="5 4"' if name == "twin" else ""
        out.append(f'<polyline fill="none" stroke="{col}" stroke-width="1.5"{dash} points="' + " ".join(f"{sx(i):.1f},{sy(v):.1f}" for i, v in enumerate(c)) + '"/>')
        out.append(f'<text x="{W - 20}" y="{36 + 14 * k}" text-anchor="end" fill="{col}">{name}</text>')
    return "\n".join(out) + "\n</svg>\n"


if __name__ == "__main__":
    raise SystemExit(main())
