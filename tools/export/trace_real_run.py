"""Real steps -> measured bundle: drive a few REAL steps of a preset, keep the LAST step's trace (steady state) and write
``<stem>.{program,annotated,webapp,measured}.json``; ``.measured.json`` holds the measured intervals beside the
simulator's prediction of the same plan and a one-line real-vs-sim parity summary.

    python tools/export/trace_real_run.py --preset llama3_8b --steps 4 --budget 60 --out runs/
    python tools/export/trace_real_run.py --preset llama3:tiny --device cpu --out /tmp/x

Reference role: ``tools/export/trace_real_run.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import _cli  # noqa: E402,F401


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", required=True)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--budget", type=float, default=None)
    ap.add_argument("--device", default="0")
    ap.add_argument("--out", default="runs")
    ap.add_argument("--name", default=None)
    a = ap.parse_args(argv)
    from dataflow_b200.core.convert import to_webapp_program
    from dataflow_b200.core.jsonio import save_program
    from dataflow_b200.lowering.planning import strip_plan_annotations
    from dataflow_b200.lowering.replay import replay_gap_pct
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    from dataflow_b200.run.presets import resolve_preset
    from dataflow_b200.run.trace_report import summarize_trace
    from dataflow_b200.runtime import trace_to_dict
    fam, cfg = resolve_preset(a.preset)
    device = None if a.device == "cpu" else int(a.device)
    tr = Trainer(fam, cfg, budget_gib=a.budget, device=device)
    for s in range(a.steps):
        tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, getattr(cfg, "vocab_size", 1024), 0, s, pin=device is not None))
    res = tr.last_result
    os.makedirs(a.out, exist_ok=True)
    stem = os.path.join(a.out, a.name or "trace-" + a.preset.replace(":", "-"))
    save_program(strip_plan_annotations(tr.program), stem + ".program.json")
    save_program(tr.program, stem + ".annotated.json")
    json.dump(to_webapp_program(tr.program), open(stem + ".webapp.json", "w"))
    rp = replay_gap_pct(tr.program, res)
    measured = {"trace": trace_to_dict(res.trace), "summary": summarize_trace(tr.program, res),
                "predicted_makespan_us": tr.planned.makespan_us, "measured_makespan_us": res.makespan_us, "replay": rp}
    json.dump(measured, open(stem + ".measured.json", "w"))
    print(f"real {res.makespan_us / 1e3:.2f} ms vs sim {tr.planned.makespan_us / 1e3:.2f} ms "
          f"(ratio {res.makespan_us / tr.planned.makespan_us:.3f}); replay gap {rp['gap_pct']:+.1f}%")
    print(f"wrote {stem}.{{program,annotated,webapp,measured}}.json")
    tr.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
