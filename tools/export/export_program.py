"""CPU-only golden path: any preset -> shaped program -> plan (+ recompute) -> simulate -> files.

    python tools/export/export_program.py --preset llama3_8b --fast-gib 60 --recompute --out examples/

Writes ``<stem>.program.json`` (bare), ``<stem>.annotated.json`` (planned), ``<stem>.webapp.json`` (the chain in the
simulator app's format) and ``<stem>.summary.json``.  Reference role: ``tools/export/export_program.py``.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from _cli import hardware_from, add_hw_flags  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", required=True)
    ap.add_argument("--fast-gib", type=float, required=True)
    ap.add_argument("--recompute", action="store_true")
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--grad-accum-rounds", type=int, default=None)
    ap.add_argument("--out", default="examples")
    ap.add_argument("--name", default=None)
    add_hw_flags(ap)
    a = ap.parse_args(argv)
    from dataflow_b200.core.convert import to_webapp_program
    from dataflow_b200.core.jsonio import program_content_id, save_program
    from dataflow_b200.lowering.flops import flop_report
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.run.driver import plan_at_budget
    from dataflow_b200.run.presets import resolve_preset
    fam, cfg = resolve_preset(a.preset)
    ov = {k: v for k, v in (("seq_len", a.seq_len), ("batch", a.batch), ("grad_accum_rounds", a.grad_accum_rounds)) if v}
    cfg = dataclasses.replace(cfg, **ov)
    hw = hardware_from(a)
    budget = int(a.fast_gib * (1 << 30))
    bare = resolve_family(fam).lower(cfg, hw=hw)
    planned = plan_at_budget(fam, cfg, budget, hw, recompute=a.recompute, leeway_bytes=None if budget >= (12 << 30) else budget // 8)
    os.makedirs(a.out, exist_ok=True)
    stem = os.path.join(a.out, a.name or a.preset.replace(":", "-"))
    save_program(bare, stem + ".program.json")
    save_program(planned.program, stem + ".annotated.json")
    json.dump(to_webapp_program(planned.program), open(stem + ".webapp.json", "w"))
    fr = flop_report(planned.program, planned.makespan_us)
    summary = {"preset": a.preset, "hardware": hw.name, "budget_gib": a.fast_gib, "policy": planned.policy,
               "makespan_ms": planned.makespan_us / 1e3, "lower_bound_ms": planned.lower_bound_us / 1e3,
               "tokens_per_s": planned.program.metadata["tokens_per_step"] / planned.makespan_us * 1e6,
               "peak_fast_gib": planned.peak_fast_bytes / 2 ** 30, "peak_backing_gib": planned.peak_backing_bytes / 2 ** 30,
               "recompute_levels": {str(k): v for k, v in planned.recompute_levels.items() if v},
               "effective_tflops": fr["effective_tflops"], "hardware_tflops": fr["hardware_tflops"],
               "program_id": program_content_id(bare), "annotated_id": program_content_id(planned.program), "transfer": planned.transfer}
    json.dump(summary, open(stem + ".summary.json", "w"), indent=1)
    print(json.dumps({k: summary[k] for k in ("makespan_ms", "tokens_per_s", "peak_fast_gib", "policy")}))
    print(f"wrote {stem}.{{program,annotated,webapp,summary}}.json")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
