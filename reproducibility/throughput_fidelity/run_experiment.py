"""Throughput fidelity study: does the simulator's predicted step time match what the engine measures, across a grid
of geometries and device budgets?

Stages (each writes a JSON file into ``--out`` and is skipped on ``--resume`` when its file exists):

    env_probe   hardware, clocks, library versions, measured copy and GEMM peaks when a GPU is present
    profile     per-task costs of the preset measured on the device (cached)
    predict     every grid cell planned and simulated (roofline costs and, after ``profile``, measured costs)
    select      the cells worth measuring: feasible, spread over the budget axis, at most ``--max-cells``
    measure     the engine runs each selected cell (warm-up excluded)
    analyze     measured / predicted per cell, geometric mean, worst cell; ``report.md`` with the table

    python reproducibility/throughput_fidelity/run_experiment.py --preset llama3_8b --seqs 4096 --t-rounds 16384 \
        --t-steps 131072 --budgets 40,60,80 --out runs/fidelity
    python reproducibility/throughput_fidelity/run_experiment.py --preset llama3:tiny --device cpu --budgets 0.02,1 --out /tmp/f

Reference role: ``reproducibility/throughput_fidelity/run_experiment.py``.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import platform
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tools"))
sys.path.insert(0, os.path.join(ROOT, "tools", "bench"))


def stage(out, name, resume, fn):
    path = os.path.join(out, name + ".json")
    if resume and os.path.exists(path):
        print(f"[{name}] kept {path}")
        return json.load(open(path))
    t0 = time.time()
    val = fn()
    json.dump(val, open(path, "w"), indent=1)
    print(f"[{name}] done in {time.time() - t0:.1f}s -> {path}")
    return val


def env_probe(device):
    import torch
    info = {"python": platform.python_version(), "torch": torch.__version__, "host": platform.node(), "device": "cpu"}
    if device is not None and torch.cuda.is_available():
        p = torch.cuda.get_device_properties(device)
        info.update(device=p.name, sms=p.multi_processor_count, memory_gib=p.total_memory / 2 ** 30)
        n = 1 << 28
        a, b = torch.empty(n, dtype=torch.uint8, device=device), torch.empty(n, dtype=torch.uint8, device=device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            b.copy_(a)
        e0.record()
        for _ in range(10):
            b.copy_(a)
        e1.record()
        torch.cuda.synchronize()
        info["copy_gbs"] = 2 * 10 * n / e0.elapsed_time(e1) / 1e6
        peaks = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(peaks):
            info["measured_peaks"] = json.load(open(peaks))
    return info


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="llama3_8b")
    ap.add_argument("--opts", default="adamw")
    ap.add_argument("--seqs", default=None)
    ap.add_argument("--t-rounds", default=None)
    ap.add_argument("--t-steps", type=int, default=None)
    ap.add_argument("--budgets", default=None, help="GiB list; or use --budget-range lo,hi with --budget-step")
    ap.add_argument("--budget-range", default=None)
    ap.add_argument("--budget-step", type=float, default=10.0)
    ap.add_argument("--max-cells", type=int, default=6)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--device", default="0")
    ap.add_argument("--out", required=True)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--stages", default="env_probe,profile,predict,select,measure,analyze")
    a = ap.parse_args(argv)
    os.makedirs(a.out, exist_ok=True)
    device = None if a.device == "cpu" else int(a.device)
    stages = a.stages.split(",")
    import predict_step
    import measure_step
    from _cli import grid_cells, hardware_from
    if a.budgets:
        budgets = a.budgets
    elif a.budget_range:
        lo, hi = (float(x) for x in a.budget_range.split(","))
        budgets = ",".join(str(lo + i * a.budget_step) for i in range(int((hi - lo) / a.budget_step) + 1))
    else:
        budgets = None
    cells_by_opt = {}
    for opt in a.opts.split(","):
        ns = argparse.Namespace(preset=a.preset, plugin=[], t_round=a.t_rounds, tokens_step=a.t_steps, ga_rounds=None, seq_len=a.seqs,
                                budget=budgets, opt=opt, dtype_policy=None, no_recompute=False, hw=None if device is not None else "b200",
                                tflops=None, bw=None, pcie=None)
        cells_by_opt[opt] = (ns, list(grid_cells(ns)))
    hw = hardware_from(next(iter(cells_by_opt.values()))[0])
    results = {}
    if "env_probe" in stages:
        results["env"] = stage(a.out, "env_probe", a.resume, lambda: env_probe(device))
    measured_costs = {}
    if "profile" in stages and device is not None:
        def prof():
            from dataflow_b200.run.driver import Trainer
            from dataflow_b200.run.profiling import profile_program
            out = {}
            for opt, (_, cells) in cells_by_opt.items():
                fam, cfg, budget = cells[0]
                tr = Trainer(fam, cfg, budget_gib=budget, device=device, init=False)
                out[opt] = profile_program(tr)
                tr.close()
            return out
        measured_costs = stage(a.out, "profile", a.resume, prof)

    def predict():
        rows = []
        for opt, (_, cells) in cells_by_opt.items():
            for fam, cfg, budget in cells:
                row, _ = predict_step.predict_cell(fam, cfg, budget, hw, True, measured_costs.get(opt))
                row["opt"] = opt
                rows.append(row)
        return rows
    pred = stage(a.out, "predict", a.resume, predict) if "predict" in stages else []

    def select():
        ok = [i for i, r in enumerate(pred) if r.get("s_step")]
        if len(ok) <= a.max_cells:
            return ok
        stride = (len(ok) - 1) / (a.max_cells - 1)
        return sorted({ok[int(round(i * stride))] for i in range(a.max_cells)})
    chosen = stage(a.out, "select", a.resume, select) if "select" in stages else []

    def measure():
        flat = [(opt, c) for opt, (_, cells) in cells_by_opt.items() for c in cells]
        rows = []
        for i in chosen:
            opt, (fam, cfg, budget) = flat[i]
            row = measure_step.measure_cell(fam, cfg, budget, hw, a.steps, device, True, bool(measured_costs))
            row.update(opt=opt, cell=i)
            rows.append(row)
        return rows
    meas = stage(a.out, "measure", a.resume, measure) if "measure" in stages else []
    if "analyze" in stages and meas:
        ratios = [r["ratio"] for r in meas]
        gm = math.exp(sum(math.log(x) for x in ratios) / len(ratios))
        worst = max(meas, key=lambda r: abs(math.log(r["ratio"])))
        lines = ["# Throughput fidelity", "", f"preset `{a.preset}`, {len(meas)} measured cells of {len(pred)} predicted; "
                 f"geometric mean measured / predicted = {gm:.3f}; worst cell {worst['ratio']:.3f} (budget {worst['budget']}).", "",
                 "| opt | seq | t_round | rounds | budget GiB | predicted s | measured s | ratio | tok/s | recompute % |", "|---|---|---|---|---|---|---|---|---|---|"]
        for r in meas:
            lines.append(f"| {r['opt']} | {r['seq']} | {r['t_round']} | {r['rounds']} | {r['budget']} | {r['pred_s']:.4f} | {r['meas_s']:.4f} | "
                         f"{r['ratio']:.3f} | {r['tok_s']:.0f} | {r['recomp_pct']:.1f} |")
        open(os.path.join(a.out, "report.md"), "w").write("\n".join(lines) + "\n")
        json.dump({"geomean_ratio": gm, "worst": worst}, open(os.path.join(a.out, "analyze.json"), "w"), indent=1)
        print(f"[analyze] geometric mean measured/predicted {gm:.3f}; report.md written")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
