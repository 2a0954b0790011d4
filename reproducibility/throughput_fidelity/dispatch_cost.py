#!/usr/bin/env python
"""What dispatching costs the host: microseconds of engine time per task and per transfer with nothing else to do.

Two synthetic programs on the chosen backend, both with tasks that do no work: a chain of ``--tasks`` tasks each feeding
the next (the per-task floor: ledger, allocation, launch, completion), and the same chain where every task's operand is
offloaded and fetched back between producer and consumer (adds one round trip per task: the per-transfer cost on both
lanes).  The difference per task is the dispatch cost of a round trip.  A plan whose tasks are shorter than the per-task
floor is dispatch-bound whatever the planner does.

    python reproducibility/throughput_fidelity/dispatch_cost.py --device cpu --tasks 400
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def programs(k: int, size: int = 4096):
    from dataflow_b200.core import ObjectSpec, OutputSpec, Program, TaskSpec, TransferDirective
    plain, trips = [], []
    for i in range(k):
        plain.append(TaskSpec(f"t{i}", inputs=(f"x{i}",), outputs=(OutputSpec(f"x{i + 1}", size),), releases_after=(f"x{i}",), runtime_us=1.0))
    for i in range(k):
        # x_i is consumed by t_i; its successor x_{i+1} leaves after t_i and is fetched straight back (a round trip per task)
        trips.append(TaskSpec(f"t{i}", inputs=(f"x{i}",), outputs=(OutputSpec(f"x{i + 1}", size),), releases_after=(f"x{i}",),
                              offload_after=(TransferDirective(f"x{i + 1}"),), prefetch_after=(TransferDirective(f"x{i + 1}"),), runtime_us=1.0))
    init = (ObjectSpec("x0", size, "fast"),)
    final = {f"x{k}": "fast"}
    bw = 1 << 20                                                  # bytes per microsecond: the copies themselves cost next to nothing
    return (Program(name=f"chain{k}", initial_objects=init, tasks=tuple(plain), final_locations=final),
            Program(name=f"trips{k}", initial_objects=init, tasks=tuple(trips), final_locations=final,
                    bandwidth_from_slow=bw, bandwidth_to_slow=bw))


def wall_per_task(engine, program, reps: int) -> float:
    engine.execute(program).raise_if_failed()                      # warm-up: pools and caches
    t0 = time.perf_counter()
    for _ in range(reps):
        engine.execute(program).raise_if_failed()
    return (time.perf_counter() - t0) / reps / len(program.tasks) * 1e6


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--device", default="cpu", help="cpu, fake (virtual time) or a CUDA ordinal")
    ap.add_argument("--tasks", type=int, default=400)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    from dataflow_b200.runtime import CpuBackend, Engine, FakeBackend
    if a.device == "fake":
        backend = FakeBackend()
    elif a.device == "cpu":
        backend = CpuBackend()
    else:
        from dataflow_b200.runtime import CudaBackend
        backend = CudaBackend(int(a.device), "poll")
    plain, trips = programs(a.tasks)
    eng = Engine(backend)
    per_task = wall_per_task(eng, plain, a.reps)
    per_task_trip = wall_per_task(eng, trips, a.reps)
    res = {"backend": a.device, "tasks": a.tasks, "us_per_task": per_task, "us_per_task_with_round_trip": per_task_trip,
           "us_per_round_trip": per_task_trip - per_task}
    print(json.dumps(res))
    if a.json:
        with open(a.json, "w") as f:
            json.dump(res, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
