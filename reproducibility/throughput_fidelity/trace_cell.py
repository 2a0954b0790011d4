#!/usr/bin/env python
"""One cell of the study, traced: plan it, run it for a few steps, and say where the last step's time went.

Writes into ``--out``: the measured trace (``<name>.measured.json``, which the simulator page overlays on its
prediction), a Chrome-trace file of the same step, and ``<name>.analysis.json`` with the predicted and measured step time,
the compute / copy overlap, the gaps of the compute lane by cause, and the audit of task costs by kind.

    python reproducibility/throughput_fidelity/trace_cell.py --preset llama3_8b --budget 60 --device 0 --out runs/cell60
    python reproducibility/throughput_fidelity/trace_cell.py --preset llama3:tiny --budget 0.02 --device cpu --out /tmp/cell
"""
from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(HERE, "diagnostics"))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="llama3:tiny")
    ap.add_argument("--budget", type=float, default=None)
    ap.add_argument("--device", default="0")
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--out", required=True)
    ap.add_argument("--name", default=None)
    a = ap.parse_args(argv)
    from task_cost_audit import audit
    from trace_overlap import gap_report, overlap_report
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    from dataflow_b200.run.presets import resolve_preset
    os.makedirs(a.out, exist_ok=True)
    fam, cfg = resolve_preset(a.preset)
    device = None if a.device == "cpu" else int(a.device)
    name = a.name or f"{a.preset.replace(':', '_')}_{a.budget if a.budget is not None else 'full'}"
    leeway = None if a.budget is None or a.budget >= 12 else int(a.budget * (1 << 30)) // 8
    tr = Trainer(fam, cfg, budget_gib=a.budget, device=device, leeway_bytes=leeway)
    try:
        vocab = getattr(cfg, "vocab_size", 1024)
        for s in range(max(a.steps, 2)):
            tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, vocab, 0, s, pin=device is not None))
        res = tr.last_result
        trace = res.trace
        ana = {"preset": a.preset, "budget_gib": a.budget, "predicted_makespan_us": tr.planned.makespan_us, "measured_makespan_us": res.makespan_us,
               "ratio": res.makespan_us / tr.planned.makespan_us, "policy": tr.planned.policy, "peak_fast_gib": res.peak_fast_bytes / 2 ** 30,
               "slab_overflows": res.slab_overflows, "overlap": overlap_report(trace), "gaps": gap_report(tr.program, trace),
               "task_costs": audit(tr.program, trace)}
        measured = {"predicted_makespan_us": tr.planned.makespan_us, "measured_makespan_us": res.makespan_us,
                    "trace": {"intervals": [{"name": i.name, "track": i.track, "start_us": i.start_us, "end_us": i.end_us} for i in trace.intervals]}}
        chrome = {"traceEvents": [{"name": i.name, "cat": i.track, "ph": "X", "ts": i.start_us, "dur": i.end_us - i.start_us, "pid": 0,
                                   "tid": {"compute": 0, "from_slow": 1, "to_slow": 2}.get(i.track, 3)} for i in trace.intervals]}
    finally:
        tr.close()
    for suffix, doc in ((".measured.json", measured), (".chrome.json", chrome), (".analysis.json", ana)):
        with open(os.path.join(a.out, name + suffix), "w") as f:
            json.dump(doc, f, indent=1)
    o = ana["overlap"]
    print(f"{name}: predicted {ana['predicted_makespan_us'] / 1e3:.2f} ms, measured {ana['measured_makespan_us'] / 1e3:.2f} ms (ratio {ana['ratio']:.3f}); "
          f"compute busy {o['compute_busy_pct']:.1f} %, copies hidden under compute: from host {o['lanes']['from_slow']['hidden_under_compute_pct']:.0f} %, "
          f"to host {o['lanes']['to_slow']['hidden_under_compute_pct']:.0f} %; gaps {ana['gaps']['idle_pct']:.1f} % of the step")
    return 0


if __name__ == "__main__":
    sys.exit(main())
