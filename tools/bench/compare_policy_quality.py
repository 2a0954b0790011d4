"""Planner quality gate (CPU): every registered policy on a corpus of lowered training programs at several budgets —
makespan over the compute-only lower bound, peak memory against the cap, planning time.

    python tools/bench/compare_policy_quality.py --presets llama3:tiny,gpt2:tiny --fractions 0.4,0.6,0.9

A budget is given as a fraction of the program's all-resident peak.  Exit code 1 if any policy exceeds its cap.
Reference role: ``tools/bench/compare_pressurefit_quality.py`` (there: two source versions of one planner on the same
corpus; here: the registered policies against each other).
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from dataclasses import replace

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from _cli import table  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--presets", default="llama3:tiny,gpt2:tiny")
    ap.add_argument("--fractions", default="0.4,0.6,0.9")
    ap.add_argument("--policies", default="pressurefit,lookahead,sliding_window,belady_reactive")
    a = ap.parse_args(argv)
    from dataflow_b200.core.convert import to_sim_chain
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.run.presets import resolve_preset
    from dataflow_b200.sim.policies import get_all_policies
    from dataflow_b200.sim.simulator import run as simulate
    pols = get_all_policies()
    rows, broke = [], 0
    for preset in a.presets.split(","):
        fam, cfg = resolve_preset(preset)
        chain = to_sim_chain(resolve_family(fam).lower(cfg), with_directives=False)
        chain = replace(chain, tasks=[replace(t, workspace_bytes=0) for t in chain.tasks])
        full = simulate(pols["all_resident"](replace(chain, fast_memory_capacity=None), None), validate=False)
        lower = sum(t.runtime for t in chain.tasks)
        for frac in [float(x) for x in a.fractions.split(",")]:
            cap = int(full.peak_fast_memory_bytes * frac)
            for name in a.policies.split(","):
                t0 = time.perf_counter()
                try:
                    log = simulate(pols[name](replace(chain, fast_memory_capacity=cap), cap), validate=False)
                    over = log.peak_fast_memory_bytes > cap
                    broke += over
                    rows.append({"preset": preset, "frac": frac, "policy": name, "x_lower": log.makespan / lower,
                                 "peak_frac": log.peak_fast_memory_bytes / cap, "plan_s": time.perf_counter() - t0,
                                 "note": "OVER CAP" if over else ""})
                except Exception as e:
                    rows.append({"preset": preset, "frac": frac, "policy": name, "plan_s": time.perf_counter() - t0,
                                 "note": f"no plan ({type(e).__name__})"})
    print(table(rows, [("preset", "{}"), ("frac", "{:.2f}"), ("policy", "{}"), ("x_lower", "{:.3f}"), ("peak_frac", "{:.3f}"),
                       ("plan_s", "{:.2f}"), ("note", "{}")]))
    return 1 if broke else 0


if __name__ == "__main__":
    raise SystemExit(main())
