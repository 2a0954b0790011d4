"""Throughput fidelity study: does the simulator's predicted step time match what the engine measures, across a grid
of geometries and device budgets?

Stages (each writes a JSON file into ``--out`` and is skipped on ``--resume`` when its file exists):

    env_probe   versions, the device, its clocks as found (read only), measured copy / GEMM / host-link rates  (stages/env_probe.py)
    profile     per-task costs of the preset measured on the device (cached)
    predict     every grid cell planned and simulated (roofline costs and, after ``profile``, measured costs)
    select      the cells worth measuring: feasible, every geometry, both ends of the budget axis, then the widest
                gaps in predicted link occupancy, at most ``--max-cells``                                        (stages/select_cells.py)
    measure     the engine runs each selected cell (warm-up excluded); rows land in ``measure.jsonl`` one by one, with the
                clocks sampled while the cell ran; ``--resume`` measures only what is missing                    (stages/sweep.py)
    analyze     measured / predicted: overall, by axis, by what the plan is bound by; causes for cells off by > 10 %  (stages/analyze.py)
    report      ``report.md``, three figures as SVG, ``report.html`` with everything inline                     (stages/make_plots.py, report.py)

Beside the study: ``diagnostics/`` (host-link calibration, GEMM burst against sustained, throttle probe, task-cost audit,
compute / copy overlap of a traced step), ``dispatch_cost.py`` (what dispatching a task and a transfer costs the host),
``trace_cell.py`` (one cell traced and analysed).

    python reproducibility/throughput_fidelity/run_experiment.py --preset llama3_8b --seqs 4096 --t-rounds 16384 \
        --t-steps 131072 --budgets 40,60,80 --out runs/fidelity
    python reproducibility/throughput_fidelity/run_experiment.py --preset llama3:tiny --device cpu --budgets 0.02,1 --out /tmp/f

Reference role: ``reproducibility/throughput_fidelity/run_experiment.py``.
"""
from __future__ import annotations

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tools"))
sys.path.insert(0, os.path.join(ROOT, "tools", "bench"))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from stages.analyze import analyze  # noqa: E402
from stages.common import stage  # noqa: E402
from stages.env_probe import env_probe  # noqa: E402
from stages.make_plots import make_plots  # noqa: E402
from stages.report import report_html, report_md  # noqa: E402
from stages.select_cells import select_cells  # noqa: E402
from stages.sweep import sweep  # noqa: E402


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
    ap.add_argument("--host-share", type=float, default=None,
                    help="share of the host link this device gets (0-1]: predictions price transfers at that share (a device whose "
                         "neighbours stream over the same host memory does not get the whole link)")
    ap.add_argument("--backing-gib", type=float, default=None,
                    help="host memory available to the run: cells whose plan needs more backing memory than this are predicted but not measured")
    ap.add_argument("--max-cells", "--target-cells", dest="max_cells", type=int, default=6)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--device", default="0")
    ap.add_argument("--out", "--results", dest="out", required=True)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--stages", default="env_probe,profile,predict,select,measure,analyze,report")
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
    if a.host_share:
        if not 0.0 < a.host_share <= 1.0:
            ap.error("--host-share is a share of the link: give a value in (0, 1]")
        import dataclasses
        hw = dataclasses.replace(hw, h2d_gbs=hw.h2d_gbs * a.host_share, d2h_gbs=hw.d2h_gbs * a.host_share, link_gbs=hw.link_gbs or hw.h2d_gbs)
    flat = [(opt, c) for opt, (_, cells) in cells_by_opt.items() for c in cells]
    env = stage(a.out, "env_probe", a.resume, lambda: env_probe(device, ROOT)) if "env_probe" in stages else {}
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
        for opt, (fam, cfg, budget) in flat:
            row, _ = predict_step.predict_cell(fam, cfg, budget, hw, True, measured_costs.get(opt))
            row["opt"] = opt
            rows.append(row)
        return rows
    pred = stage(a.out, "predict", a.resume, predict) if "predict" in stages else []
    def choose():
        usable = pred
        if a.backing_gib is not None:          # a plan that needs more host memory than the run may use is not measured
            usable = [r if r.get("backing_gib", 0.0) <= a.backing_gib else {**r, "s_step": None, "note": "needs more backing memory"} for r in pred]
        return select_cells(usable, a.max_cells)
    chosen = stage(a.out, "select", a.resume, choose) if "select" in stages else []
    meas = []
    if "measure" in stages:
        def one(fam, cfg, budget):
            return measure_step.measure_cell(fam, cfg, budget, hw, a.steps, device, True, bool(measured_costs))
        one.device = device
        meas = sweep(a.out, flat, chosen, one, a.resume)
    ana = {}
    if "analyze" in stages and meas:
        ana = stage(a.out, "analyze", False, lambda: analyze(pred, meas))
        if ana.get("cells"):
            print(f"[analyze] geometric mean measured/predicted {ana['geomean_ratio']:.3f} over {ana['cells']} cells; "
                  f"{100 * ana['within_10pct']:.0f} % within 10 %")
    if ("report" in stages or "analyze" in stages) and meas:
        plots = make_plots(meas)
        for name, svg in plots.items():
            with open(os.path.join(a.out, name), "w") as f:
                f.write(svg)
        md = report_md(a.preset, env, pred, meas, ana or analyze(pred, meas))
        with open(os.path.join(a.out, "report.md"), "w") as f:
            f.write(md)
        with open(os.path.join(a.out, "report.html"), "w") as f:
            f.write(report_html(md, plots))
        print(f"[report] report.md, report.html and {len(plots)} figures written to {a.out}")
    return 0 if not meas or any("ratio" in m for m in meas) else 1


if __name__ == "__main__":
    raise SystemExit(main())
