"""The simulator on the command line, for task chains saved as JSON (``TaskChain.save`` / the export tools).

    python -m dataflow_b200.sim validate chain.json [--planning-input]       every problem of the first failing stage, by rule
    python -m dataflow_b200.sim plan     chain.json --policy min_grow --capacity-gib 40 [-o planned.json]
    python -m dataflow_b200.sim simulate planned.json [--stalls]            makespan, peaks, lane use; the stall report
    python -m dataflow_b200.sim compare  chain.json --capacity-gib 40 [--policies a,b,c]     one row per planner

Exit code 0 when the chain is valid / a plan was found / the run completed, 1 otherwise.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from dataclasses import replace

from . import build_stall_report, run
from .policies import get_all_policies
from .schema import TaskChain
from .validate import RULES, STAGES


def _cap(a) -> int | None:
    return int(a.capacity_gib * (1 << 30)) if a.capacity_gib is not None else None


def cmd_validate(a) -> int:
    chain = TaskChain.load(a.chain)
    stages = ("ids", "capacity") if a.planning_input else ("ids", "transfers", "lifetimes", "capacity")
    for name in stages:
        found = STAGES[name](chain)
        print(f"{name:<10} {'ok' if not found else f'{len(found)} problem(s)'}")
        for p in found:
            print(f"  {p}    [{RULES.get(p.rule, '')}]")
        if found:
            return 1
    if a.planning_input:
        carrying = next((t.id for t in chain.tasks if t.releases_after or t.offload_after or t.prefetch_after), None)
        if carrying is not None:
            print(f"already-planned: task {carrying!r} carries releases or transfers; planners take a bare chain")
            return 1
    print(f"valid: {len(chain.tasks)} tasks, {len(chain.sizes())} objects")
    return 0


def cmd_plan(a) -> int:
    chain = TaskChain.load(a.chain)
    pols = get_all_policies()
    if a.policy not in pols:
        print(f"unknown policy {a.policy!r}; known: {', '.join(sorted(pols))}", file=sys.stderr)
        return 1
    cap = _cap(a) if a.capacity_gib is not None else chain.fast_memory_capacity
    t0 = time.perf_counter()
    try:
        planned = pols[a.policy](replace(chain, fast_memory_capacity=cap), cap)
    except Exception as e:      # noqa: BLE001  (a planner's refusal is the answer)
        print(f"{a.policy}: no plan ({type(e).__name__}: {e})", file=sys.stderr)
        return 1
    log = run(planned)
    lower = sum(t.runtime for t in chain.tasks)
    print(f"{a.policy}: makespan {log.makespan:.0f} us = {log.makespan / max(lower, 1e-9):.3f} x compute-only, peak fast {log.peak_fast_memory_bytes / 2 ** 30:.3f} GiB, "
          f"{len(log.transfer_intervals('from_slow'))} fetches, {len(log.transfer_intervals('to_slow'))} offloads, planned in {time.perf_counter() - t0:.2f} s")
    if a.output:
        planned.save(a.output)
        print(f"wrote {a.output}")
    return 0


def cmd_simulate(a) -> int:
    chain = TaskChain.load(a.chain)
    try:
        log = run(chain)
    except ValueError as e:
        print(f"{type(e).__name__}: {e}", file=sys.stderr)
        return 1
    busy = {d: sum(iv.end - iv.start for iv in log.transfer_intervals(d)) for d in ("from_slow", "to_slow")}
    out = {"makespan_us": log.makespan, "peak_fast_bytes": log.peak_fast_memory_bytes, "peak_backing_bytes": log.peak_backing_memory_bytes,
           "stall_us": sum(log.stalls.values()), "stalled_tasks": len(log.stalls),
           "lane_busy_pct": {d: 100.0 * v / log.makespan if log.makespan else 0.0 for d, v in busy.items()}}
    print(json.dumps(out))
    if a.stalls:
        print(build_stall_report(chain, log).format(a.top))
    return 0


def cmd_compare(a) -> int:
    chain = TaskChain.load(a.chain)
    pols = get_all_policies()
    names = a.policies.split(",") if a.policies else sorted(pols)
    cap = _cap(a) if a.capacity_gib is not None else chain.fast_memory_capacity
    lower = sum(t.runtime for t in chain.tasks)
    rows = []
    for name in names:
        t0 = time.perf_counter()
        try:
            log = run(pols[name](replace(chain, fast_memory_capacity=cap), cap))
            rows.append((log.makespan, name, f"{log.makespan:>14.0f} us  {log.makespan / max(lower, 1e-9):7.3f} x  peak {log.peak_fast_memory_bytes / 2 ** 30:8.3f} GiB  "
                                             f"{time.perf_counter() - t0:6.2f} s"))
        except Exception as e:  # noqa: BLE001
            rows.append((float("inf"), name, f"no plan ({type(e).__name__})"))
    for _, name, line in sorted(rows):
        print(f"{name:<16} {line}")
    return 0 if any(r[0] < float("inf") for r in rows) else 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dataflow_b200.sim", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    v = sub.add_parser("validate")
    v.add_argument("chain")
    v.add_argument("--planning-input", action="store_true")
    p = sub.add_parser("plan")
    p.add_argument("chain")
    p.add_argument("--policy", default="pressurefit")
    p.add_argument("--capacity-gib", type=float, default=None)
    p.add_argument("-o", "--output", default=None)
    s = sub.add_parser("simulate")
    s.add_argument("chain")
    s.add_argument("--stalls", action="store_true")
    s.add_argument("--top", type=int, default=10)
    c = sub.add_parser("compare")
    c.add_argument("chain")
    c.add_argument("--capacity-gib", type=float, default=None)
    c.add_argument("--policies", default=None)
    a = ap.parse_args(argv)
    return {"validate": cmd_validate, "plan": cmd_plan, "simulate": cmd_simulate, "compare": cmd_compare}[a.cmd](a)


if __name__ == "__main__":
    raise SystemExit(main())
