"""Simulated throughput sweeps (CPU, seconds): lower the true program of a preset, plan every cell of the grid and
read the simulator-verified schedule back as a table.

    python tools/bench/predict_step.py --preset llama3_8b --budget 40,60,80 --tokens-step 131072 --t-round 16384
    python tools/bench/predict_step.py --preset llama3:tiny --top 8          # single point: the most expensive tasks

Columns: s/step, tokens/s, effective / hardware TFLOP/s, device and host peaks, host-link bytes and busy share,
recompute and idle share, ETA for --steps.  ``--measured`` prices tasks with profiled costs (needs the GPU once per
geometry; cached on disk).  Reference role: ``tools/bench/predict_step.py``.
"""
from __future__ import annotations

import argparse
import dataclasses
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from _cli import add_grid_flags, add_hw_flags, grid_cells, hardware_from, table  # noqa: E402


def predict_cell(fam, cfg, budget_gib, hw, recompute=True, measured=None):
    from dataflow_b200.core.convert import to_sim_chain
    from dataflow_b200.lowering.flops import flop_report
    from dataflow_b200.run.driver import plan_at_budget
    from dataflow_b200.sim.simulator import run as simulate
    budget = None if budget_gib is None else int(budget_gib * (1 << 30))
    row = {"seq": cfg.seq_len, "t_round": cfg.seq_len * cfg.batch, "rounds": cfg.grad_accum_rounds, "budget": budget_gib}
    try:
        # the leeway share of small budgets scales down with them
        leeway = None if budget is None or budget >= (12 << 30) else budget // 8
        planned = plan_at_budget(fam, cfg, budget, hw, recompute=recompute, measured=measured, leeway_bytes=leeway)
    except Exception as e:                                          # an infeasible cell is a row, not a crash
        row["note"] = f"INFEASIBLE ({type(e).__name__})"
        return row, None
    # workspace is accounted outside the object pool: simulate the objects alone, as the planner did
    chain = to_sim_chain(planned.program)
    chain = dataclasses.replace(chain, tasks=[dataclasses.replace(t, workspace_bytes=0) for t in chain.tasks])
    log = simulate(chain, validate=False)
    fr = flop_report(planned.program, planned.makespan_us)
    tokens = planned.program.metadata["tokens_per_step"]
    busy = sum(iv.end - iv.start for iv in log.compute_intervals())
    rec = sum(iv.end - iv.start for iv in log.compute_intervals() if "recompute" in iv.task_id)
    h2d = sum(iv.end - iv.start for iv in log.transfer_intervals("from_slow"))
    d2h = sum(iv.end - iv.start for iv in log.transfer_intervals("to_slow"))
    sizes = planned.program.object_sizes()
    moved = sum(sizes.get(iv.task_id.split(":", 1)[-1], 0) for iv in log.transfer_intervals())
    row.update(s_step=planned.makespan_us / 1e6, tok_s=tokens / planned.makespan_us * 1e6, eff_tf=fr["effective_tflops"],
               hw_tf=fr["hardware_tflops"], fast_gib=planned.peak_fast_bytes / 2 ** 30, backing_gib=planned.peak_backing_bytes / 2 ** 30,
               link_gb=moved / 1e9, link_pct=100.0 * max(h2d, d2h) / planned.makespan_us, recomp_pct=100.0 * rec / max(busy, 1e-9),
               idle_pct=100.0 * planned.idle_fraction, policy=planned.policy, note="")
    return row, planned


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_grid_flags(ap)
    add_hw_flags(ap)
    ap.add_argument("--measured", action="store_true", help="profiled task costs instead of the roofline seeds")
    ap.add_argument("--steps", type=int, default=None, help="print an ETA column for this many steps")
    ap.add_argument("--top", type=int, default=0, help="single point: list the N most expensive tasks")
    ap.add_argument("--json", default=None, help="also write the rows to this file")
    a = ap.parse_args(argv)
    hw = hardware_from(a)
    rows, last = [], None
    for fam, cfg, budget in grid_cells(a):
        measured = None
        if a.measured:
            from dataflow_b200.run.driver import Trainer
            from dataflow_b200.run.profiling import profile_program
            tr = Trainer(fam, cfg, budget_gib=budget, device=0, hw=hw, recompute=not a.no_recompute, init=False)
            measured = profile_program(tr)
            tr.close()
        row, planned = predict_cell(fam, cfg, budget, hw, not a.no_recompute, measured)
        if a.steps and row.get("s_step"):
            row["eta_h"] = row["s_step"] * a.steps / 3600
        rows.append(row)
        last = planned or last
    cols = [("seq", "{}"), ("t_round", "{}"), ("rounds", "{}"), ("budget", "{:.1f}"), ("s_step", "{:.3f}"), ("tok_s", "{:.0f}"),
            ("eff_tf", "{:.1f}"), ("hw_tf", "{:.1f}"), ("fast_gib", "{:.2f}"), ("backing_gib", "{:.2f}"), ("link_gb", "{:.1f}"),
            ("link_pct", "{:.0f}"), ("recomp_pct", "{:.1f}"), ("idle_pct", "{:.1f}"), ("policy", "{}")]
    if a.steps:
        cols.append(("eta_h", "{:.1f}"))
    cols.append(("note", "{}"))
    print(f"hardware: {hw.name} ({hw.peak_tflops:.0f} TFLOP/s bf16, {hw.hbm_gbs:.0f} GB/s, host link {hw.h2d_gbs:.0f}/{hw.d2h_gbs:.0f} GB/s)")
    print(table(rows, cols))
    if a.top and last is not None:
        tasks = sorted(last.program.tasks, key=lambda t: -t.runtime_us)[:a.top]
        print(f"\n{a.top} most expensive tasks of the last cell:")
        print(table([{"task": t.id, "ms": t.runtime_us / 1e3, "ws_mib": t.workspace_bytes / 2 ** 20} for t in tasks],
                    [("task", "{}"), ("ms", "{:.3f}"), ("ws_mib", "{:.0f}")]))
    if a.json:
        import json
        json.dump(rows, open(a.json, "w"), indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
