"""Gap census: where the compute lane of a REAL step sat idle, from the run's own interval trace.

    python tools/bench/gap_census.py --preset llama3:tiny --device cpu --steps 4
    python tools/bench/gap_census.py --trace run.trace.json --program run.annotated.json

Every gap between consecutive compute intervals is attributed to the task that followed it and classified: *transfer*
(an input of that task was still arriving on the host link when the previous task ended), *dispatch* (everything was
present; the engine had not launched yet) — with the distribution (p50 / p90 / max), the total per class and the ten
largest gaps.  Reference role: ``tools/bench/gap_census.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import _cli  # noqa: E402,F401


def census(program, trace, floor_us: float = 0.0) -> dict:
    by_id = {t.id: t for t in program.tasks}
    comp = sorted(trace.by_track("compute"), key=lambda i: i.start_us)
    arrivals = {}
    for iv in trace.by_track("from_slow"):
        arrivals[iv.name] = max(arrivals.get(iv.name, 0.0), iv.end_us)
    rows = []
    for a, b in zip(comp[:-1], comp[1:]):
        gap = b.start_us - a.end_us
        if gap <= floor_us:
            continue
        t = by_id.get(b.name)
        late = [i for i in (t.inputs if t else ()) if arrivals.get(i, -1.0) > a.end_us]
        rows.append({"gap_us": gap, "before": b.name, "after": a.name, "cause": "transfer" if late else "dispatch", "late_inputs": late})
    gaps = sorted(r["gap_us"] for r in rows)
    pct = lambda q: gaps[min(int(len(gaps) * q), len(gaps) - 1)] if gaps else 0.0  # noqa: E731
    total = {c: sum(r["gap_us"] for r in rows if r["cause"] == c) for c in ("transfer", "dispatch")}
    span = comp[-1].end_us - comp[0].start_us if comp else 0.0
    return {"intervals": len(comp), "gaps": len(rows), "p50_us": pct(0.5), "p90_us": pct(0.9), "max_us": gaps[-1] if gaps else 0.0,
            "total_us": total, "span_us": span, "idle_pct": 100.0 * sum(total.values()) / span if span else 0.0,
            "largest": sorted(rows, key=lambda r: -r["gap_us"])[:10]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--trace", default=None, help="a saved run trace (JSON); needs --program")
    ap.add_argument("--program", default=None, help="the annotated program the trace came from")
    ap.add_argument("--preset", default="llama3:tiny")
    ap.add_argument("--device", default="0")
    ap.add_argument("--budget", type=float, default=None)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--floor-us", type=float, default=0.0, help="ignore gaps at or below this")
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    if a.trace:
        from dataflow_b200.core.jsonio import load_program
        from dataflow_b200.runtime import trace_from_dict
        program = load_program(a.program)
        trace = trace_from_dict(json.load(open(a.trace)))
    else:
        from dataflow_b200.run.driver import Trainer, synthetic_rounds
        from dataflow_b200.run.presets import resolve_preset
        fam, cfg = resolve_preset(a.preset)
        device = None if a.device == "cpu" else int(a.device)
        tr = Trainer(fam, cfg, budget_gib=a.budget, device=device)
        for s in range(a.steps):
            tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, getattr(cfg, "vocab_size", 1024), 0, s, pin=device is not None))
        program, trace = tr.program, tr.last_result.trace
        tr.close()
    c = census(program, trace, a.floor_us)
    print(f"{c['intervals']} compute intervals, {c['gaps']} gaps: p50 {c['p50_us']:.1f} us, p90 {c['p90_us']:.1f} us, max {c['max_us']:.1f} us; "
          f"idle {c['idle_pct']:.1f}% of the span ({c['total_us']['transfer'] / 1e3:.2f} ms waiting for transfers, "
          f"{c['total_us']['dispatch'] / 1e3:.2f} ms dispatch)")
    for r in c["largest"]:
        print(f"  {r['gap_us']:10.1f} us  before {r['before']:<28} ({r['cause']}{': ' + ','.join(r['late_inputs'][:3]) if r['late_inputs'] else ''})")
    if a.json:
        json.dump(c, open(a.json, "w"), indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
