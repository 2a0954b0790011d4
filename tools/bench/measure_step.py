"""Measured throughput sweeps (GPU, minutes): the same grid as ``predict_step.py``; each cell RUNS the engine and reports
the warmed measurement beside the plan's prediction — pred_s, meas_s, ratio, tokens/s, effective / hardware TFLOP/s,
recompute share, replay gap.

    python tools/bench/measure_step.py --preset llama3_8b --budget 60 --tokens-step 131072 --t-round 16384 --steps 6

The first 3 steps of a cell are warm-up and excluded from the mean.  ``--device cpu`` runs the host backend (tiny
presets).  Reference role: ``tools/bench/measure_step.py``.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from _cli import add_grid_flags, add_hw_flags, grid_cells, hardware_from, table  # noqa: E402


def measure_cell(fam, cfg, budget, hw, steps, device, recompute, measured_plan, warmup=3):
    from dataflow_b200.lowering.flops import flop_report
    from dataflow_b200.lowering.replay import replay_gap_pct
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    row = {"seq": cfg.seq_len, "t_round": cfg.seq_len * cfg.batch, "rounds": cfg.grad_accum_rounds, "budget": budget}
    leeway = None if budget is None or budget >= 12 else int(budget * (1 << 30)) // 8
    tr = Trainer(fam, cfg, budget_gib=budget, device=device, hw=hw if device is not None else None, recompute=recompute,
                 profile=measured_plan and device is not None, leeway_bytes=leeway,
                 lower_kwargs={"resident_params": True} if device is not None else None)
    try:
        vocab = getattr(cfg, "vocab_size", 1024)
        times = []
        for s in range(max(steps, warmup + 1)):
            tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, vocab, 0, s, pin=device is not None))
            if s >= warmup:
                times.append(tr.last_result.makespan_us)
        meas = sum(times) / len(times)
        fr = flop_report(tr.program, meas)
        tokens = tr.program.metadata["tokens_per_step"]
        rp = replay_gap_pct(tr.program, tr.last_result)
        row.update(pred_s=tr.planned.makespan_us / 1e6, meas_s=meas / 1e6, ratio=meas / tr.planned.makespan_us,
                   tok_s=tokens / meas * 1e6, eff_tf=fr["effective_tflops"], hw_tf=fr["hardware_tflops"],
                   recomp_pct=100.0 * fr["recompute_flops"] / max(fr["hardware_flops"], 1.0), replay_gap_pct=rp["gap_pct"],
                   peak_gib=tr.last_result.peak_fast_bytes / 2 ** 30, overflows=tr.last_result.slab_overflows)
    finally:
        tr.close()
    return row


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_grid_flags(ap)
    add_hw_flags(ap)
    ap.add_argument("--steps", type=int, default=6, help="steps per cell (first 3 are warm-up)")
    ap.add_argument("--device", default="0", help="CUDA device index, or 'cpu'")
    ap.add_argument("--measured-plan", action="store_true", help="plan from profiled task costs")
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    device = None if a.device == "cpu" else int(a.device)
    hw = hardware_from(a)
    rows = []
    for fam, cfg, budget in grid_cells(a):
        rows.append(measure_cell(fam, cfg, budget, hw, a.steps, device, not a.no_recompute, a.measured_plan))
    print(table(rows, [("seq", "{}"), ("t_round", "{}"), ("rounds", "{}"), ("budget", "{:.1f}"), ("pred_s", "{:.4f}"), ("meas_s", "{:.4f}"),
                       ("ratio", "{:.2f}"), ("tok_s", "{:.0f}"), ("eff_tf", "{:.1f}"), ("hw_tf", "{:.1f}"), ("recomp_pct", "{:.1f}"),
                       ("replay_gap_pct", "{:+.1f}"), ("peak_gib", "{:.2f}"), ("overflows", "{}")]))
    if a.json:
        import json
        json.dump(rows, open(a.json, "w"), indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
