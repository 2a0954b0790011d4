"""Dispatch floor of the executor: K trivial tasks in a chain, no transfers; the step time divided by K is what one task
costs in pure engine overhead (graph walk, ledger, launch call, completion tracking).

    python tools/bench/dispatch_floor.py --backend fake --tasks 2000
    python tools/bench/dispatch_floor.py --backend cuda --tasks 2000 --spin-us 20      # inter-kernel gap on a device

With ``--spin-us`` every task launches the calibrated spin kernel, and the report also gives the median gap between
consecutive kernels on the compute stream.  Reference role: ``tools/bench/dispatch_floor.py``.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import _cli  # noqa: E402,F401  (puts the repository root on the path)


def chain_program(k: int, runtime_us: float):
    from dataflow_b200.core.program import OutputSpec, Program, TaskSpec
    tasks = []
    for i in range(k):
        tasks.append(TaskSpec(id=f"t{i}", inputs=() if i == 0 else (f"x{i}",), outputs=(OutputSpec(f"x{i + 1}", 256),),
                              runtime_us=runtime_us, compute_block_key="noop", releases_after=() if i == 0 else (f"x{i}",)))
    return Program(name=f"floor{k}", tasks=tuple(tasks), final_locations={f"x{k}": "fast"})


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--backend", default="fake", choices=["fake", "cpu", "cuda"])
    ap.add_argument("--tasks", type=int, default=2000)
    ap.add_argument("--spin-us", type=float, default=0.0)
    ap.add_argument("--repeat", type=int, default=5)
    ap.add_argument("--dispatch-ahead", type=int, default=2)
    a = ap.parse_args(argv)
    from dataflow_b200.runtime import CpuBackend, Engine, FakeBackend, Session
    if a.backend == "cuda":
        from dataflow_b200.runtime import CudaBackend
        be = CudaBackend(0, "poll")
    else:
        be = FakeBackend() if a.backend == "fake" else CpuBackend()

    class Noop:
        def launch(self, ctx):
            if a.spin_us:
                ctx.backend.busy(0, a.spin_us)

    prog = chain_program(a.tasks, max(a.spin_us, 1.0))
    sess = Session(be)
    eng = Engine(be, session=sess)
    noop = Noop()
    resolver = lambda task: noop  # noqa: E731
    walls, gaps = [], []
    for r in range(a.repeat):
        t0 = time.perf_counter()
        res = eng.execute(prog, resolver, dispatch_ahead=a.dispatch_ahead if a.backend == "cuda" else 0)
        walls.append((time.perf_counter() - t0) * 1e6)
        res.raise_if_failed()
        comp = sorted(res.trace.by_track("compute"), key=lambda i: i.start_us)
        gaps = sorted(b.start_us - c.end_us for c, b in zip(comp[:-1], comp[1:]))
    best = min(walls)
    print(f"backend {a.backend}: {a.tasks} tasks, best of {a.repeat}: {best / 1e3:.2f} ms wall, {best / a.tasks:.2f} us/task host cost")
    if gaps and a.backend != "fake":
        print(f"inter-task gap on the compute lane: p50 {gaps[len(gaps) // 2]:.1f} us, p90 {gaps[int(len(gaps) * 0.9)]:.1f} us, max {gaps[-1]:.1f} us")
    print(f"dispatch_us_total (engine counter): {res.stats.get('dispatch_us_total', 0.0) / a.tasks:.2f} us/task")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
