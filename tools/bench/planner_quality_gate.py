"""Planner quality gate over a scenario corpus (CPU, no device).

A scenario = one model of the workload library x one hardware preset x one step shape (sequence length, tokens per round,
rounds) x one fast-memory budget, given as a fraction of the all-resident peak.  Every scenario is traced, priced and
realised into a task chain; every registered policy plans it; the simulator decides: a plan counts only if it
finishes under the cap.  Per policy the gate reports how many scenarios it solves, the geometric mean of
makespan / compute-only lower bound over the scenarios EVERY compared policy solves, how often it is the best, and its
planning time.  ``auto`` is what the training entry uses: the better of Lookahead and PressureFit per scenario.

    python tools/bench/planner_quality_gate.py                       # the full corpus (several hundred scenarios, minutes)
    python tools/bench/planner_quality_gate.py --quick               # a dozen scenarios (seconds; what the test suite runs)
    python tools/bench/planner_quality_gate.py --write-baseline      # record this tree's numbers as the baseline
    python tools/bench/planner_quality_gate.py --check               # exit 1 if ``auto`` regressed against the baseline

The baseline lives beside this file (``planner_quality_baseline.json``).  ``--check`` fails when a plan exceeds its cap,
when ``auto`` solves fewer scenarios than recorded, or when its geometric mean is more than 1 % worse.
Reference role: ``tools/bench/compare_pressurefit_quality.py`` (390 scenarios, valid counts, geometric means, wall time).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time
from dataclasses import replace

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))
BASELINE = os.path.join(HERE, "planner_quality_baseline.json")

POLICIES = ("lookahead", "pressurefit", "sliding_window", "belady_reactive", "roundtrip", "max_reduce", "min_grow")
SHAPES = ((4096, 16384, 2), (8192, 16384, 1))                       # (seq_len, tokens per round, rounds)
FRACTIONS = (0.25, 0.4, 0.6, 0.85)
HARDWARE = ("B200", "H100", "RTX_5090")


def corpus(quick: bool):
    from dataflow_b200.sim.workloads.builders import MODEL_LIBRARY
    models = sorted(MODEL_LIBRARY)
    if quick:
        return [(m, "B200", SHAPES[0], f) for m in ("llama3_8b", "olmoe_1b_7b", "deepseek_v3_2") for f in (0.3, 0.5, 0.8, 0.95)]
    return [(m, hw, shape, f) for m in models for hw in HARDWARE for shape in SHAPES for f in FRACTIONS]


def run_corpus(scenarios, policies=POLICIES, log=None) -> dict:
    from dataflow_b200.sim.policies import get_all_policies
    from dataflow_b200.sim.simulator import run as simulate
    from dataflow_b200.sim.workloads.builders import MODEL_LIBRARY, TrainingConfig, trace_training_model
    from dataflow_b200.sim.workloads.hardware import get_hardware
    from dataflow_b200.sim.workloads.schema import realize_workload
    pols = get_all_policies()
    chains: dict[tuple, tuple] = {}
    rows = []
    over_cap = 0
    for n, (model, hw_name, shape, frac) in enumerate(scenarios):
        key = (model, hw_name, shape)
        if key not in chains:
            prog = trace_training_model(MODEL_LIBRARY[model], TrainingConfig(seq_len=shape[0], tokens_per_round=shape[1], rounds=shape[2]))
            chain = realize_workload(prog, get_hardware(hw_name), None)
            full = simulate(pols["all_resident"](replace(chain, fast_memory_capacity=None), None), validate=False)
            chains[key] = (chain, full.peak_fast_memory_bytes, sum(t.runtime for t in chain.tasks))
        chain, peak, lower = chains[key]
        cap = int(peak * frac)
        row = {"model": model, "hw": hw_name, "seq": shape[0], "tokens": shape[1] * shape[2], "frac": frac, "cap": cap, "x": {}, "plan_s": {}}
        for name in policies:
            t0 = time.perf_counter()
            try:
                lg = simulate(pols[name](replace(chain, fast_memory_capacity=cap), cap), validate=False)
                if lg.peak_fast_memory_bytes > cap:
                    over_cap += 1
                    row["x"][name] = None
                else:
                    row["x"][name] = lg.makespan / lower
            except Exception:       # noqa: BLE001  (a policy that finds no plan)
                row["x"][name] = None
            row["plan_s"][name] = time.perf_counter() - t0
        both = [row["x"][p] for p in ("lookahead", "pressurefit") if p in row["x"] and row["x"][p] is not None]
        row["x"]["auto"] = min(both) if both else None
        row["plan_s"]["auto"] = sum(row["plan_s"].get(p, 0.0) for p in ("lookahead", "pressurefit"))
        rows.append(row)
        if log and (n + 1) % 20 == 0:
            log(f"{n + 1}/{len(scenarios)} scenarios")
    return {"rows": rows, "over_cap": over_cap}


def summarise(result: dict, policies) -> dict:
    rows = result["rows"]
    names = list(policies) + ["auto"]
    out = {"scenarios": len(rows), "over_cap": result["over_cap"], "policies": {}}
    common = [r for r in rows if all(r["x"].get(p) is not None for p in names)]
    for p in names:
        solved = [r for r in rows if r["x"].get(p) is not None]
        best = sum(1 for r in solved if r["x"][p] <= min(v for k, v in r["x"].items() if v is not None and k != "auto") * (1 + 1e-9))
        out["policies"][p] = {
            "solved": len(solved),
            "geomean_x_lower_common": math.exp(sum(math.log(r["x"][p]) for r in common) / len(common)) if common else None,
            "geomean_x_lower_solved": math.exp(sum(math.log(r["x"][p]) for r in solved) / len(solved)) if solved else None,
            "best_in": best,
            "plan_s_total": sum(r["plan_s"][p] for r in rows),
        }
    out["common_scenarios"] = len(common)
    return out


def check(summary: dict, baseline: dict, tol: float = 0.01) -> list[str]:
    problems = []
    if summary["over_cap"]:
        problems.append(f"{summary['over_cap']} plans exceeded their cap")
    if summary["scenarios"] != baseline.get("scenarios"):
        return problems + [f"corpus size changed ({baseline.get('scenarios')} -> {summary['scenarios']}): rewrite the baseline"]
    # what training uses, and the two span planners that lead the table: none may solve fewer scenarios or get worse by more than 1 %
    for name in ("auto", "min_grow", "max_reduce"):
        a, b = summary["policies"].get(name), baseline["policies"].get(name)
        if not a or not b:
            continue
        if a["solved"] < b["solved"]:
            problems.append(f"{name} solves {a['solved']} scenarios, the baseline {b['solved']}")
        if a["geomean_x_lower_solved"] and b["geomean_x_lower_solved"] and a["geomean_x_lower_solved"] > b["geomean_x_lower_solved"] * (1 + tol):
            problems.append(f"{name}'s geometric mean got worse: {b['geomean_x_lower_solved']:.4f} -> {a['geomean_x_lower_solved']:.4f}")
    return problems


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--policies", default=",".join(POLICIES))
    ap.add_argument("--write-baseline", action="store_true")
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--json", default=None, help="write the per-scenario rows and the summary here")
    a = ap.parse_args(argv)
    from _cli import table
    policies = tuple(p for p in a.policies.split(",") if p)
    scen = corpus(a.quick)
    t0 = time.perf_counter()
    result = run_corpus(scen, policies, log=lambda s: print(s, file=sys.stderr, flush=True))
    summary = summarise(result, policies)
    summary["wall_s"] = time.perf_counter() - t0
    summary["corpus"] = "quick" if a.quick else "full"
    rows = [{"policy": p, **v} for p, v in summary["policies"].items()]
    print(f"{summary['scenarios']} scenarios, {summary['common_scenarios']} solved by every policy, {summary['over_cap']} plans over their cap, "
          f"{summary['wall_s']:.0f} s")
    print(table(rows, [("policy", "{}"), ("solved", "{}"), ("geomean_x_lower_common", "{:.4f}"), ("geomean_x_lower_solved", "{:.4f}"),
                       ("best_in", "{}"), ("plan_s_total", "{:.1f}")]))
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"summary": summary, "rows": result["rows"]}, f, indent=1)
    key = summary["corpus"]
    if a.write_baseline:
        data = json.load(open(BASELINE)) if os.path.exists(BASELINE) else {}
        data[key] = summary
        with open(BASELINE, "w") as f:
            json.dump(data, f, indent=1, sort_keys=True)
        print(f"baseline [{key}] written to {BASELINE}")
    if a.check:
        if not os.path.exists(BASELINE) or key not in json.load(open(BASELINE)):
            print(f"no baseline for the {key} corpus")
            return 1
        problems = check(summary, json.load(open(BASELINE))[key])
        for p in problems:
            print("REGRESSION:", p)
        return 1 if problems else 0
    return 1 if summary["over_cap"] else 0


if __name__ == "__main__":
    raise SystemExit(main())
