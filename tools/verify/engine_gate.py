"""Real executor versus simulator prediction on a synthetic chain: every task occupies the compute stream for exactly its
planned runtime (calibrated spin kernel on a device, busy wait on the host backend), so any excess of the measured step
over the simulated one is engine overhead — and the peak device bytes must equal the simulator's exactly.

    python tools/verify/engine_gate.py --config mini --fast-gib 0.05 --backend cpu
    python tools/verify/engine_gate.py --config 8b --fast-gib 16 --backend cuda --out runs/

Configs: ``mini`` (6 layers, 2 rounds), ``small`` (16 layers), ``8b`` (32 layers shaped like an 8B model's objects and
task times).  Writes ``<out>/engine_gate-<config>.{summary,trace}.json``.  Reference role: ``tools/verify/engine_gate.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import _cli  # noqa: E402,F401

CONFIGS = {"mini": dict(layers=6, rounds=2, w=4 << 20, a=6 << 20, x=1 << 20, fwd_us=400.0, bwd_us=800.0, opt_us=200.0),
           "small": dict(layers=16, rounds=2, w=32 << 20, a=48 << 20, x=8 << 20, fwd_us=1500.0, bwd_us=3000.0, opt_us=600.0),
           "8b": dict(layers=32, rounds=2, w=436 << 20, a=700 << 20, x=128 << 20, fwd_us=9000.0, bwd_us=18000.0, opt_us=2500.0)}


def synthetic_program(c):
    from dataflow_b200.core.program import ObjectSpec, OutputSpec, Program, TaskSpec
    L, R = c["layers"], c["rounds"]
    init = [ObjectSpec(f"W_{i}", c["w"], location="backing", persistent=True) for i in range(L)]
    init += [ObjectSpec(f"O_{i}", 2 * c["w"], location="backing", persistent=True) for i in range(L)]
    tasks = []
    for r in range(R):
        tasks.append(TaskSpec(f"in_{r}", (), (OutputSpec(f"x_{r}_0", c["x"]),), runtime_us=20.0, compute_block_key="synthetic"))
        for i in range(L):
            tasks.append(TaskSpec(f"fwd_{r}_{i}", (f"x_{r}_{i}", f"W_{i}"), (OutputSpec(f"A_{r}_{i}", c["a"]), OutputSpec(f"x_{r}_{i + 1}", c["x"])),
                                  runtime_us=c["fwd_us"], compute_block_key="synthetic"))
        tasks.append(TaskSpec(f"head_{r}", (f"x_{r}_{L}",), (OutputSpec(f"g_{r}_{L}", c["x"]),), runtime_us=c["fwd_us"], compute_block_key="synthetic"))
        for i in reversed(range(L)):
            first = r == 0
            tasks.append(TaskSpec(f"bwd_{r}_{i}", (f"g_{r}_{i + 1}", f"A_{r}_{i}", f"W_{i}") + (() if first else (f"dW_{i}",)),
                                  (OutputSpec(f"g_{r}_{i}", c["x"]),) + ((OutputSpec(f"dW_{i}", c["w"]),) if first else ()),
                                  mutates=() if first else (f"dW_{i}",), runtime_us=c["bwd_us"], compute_block_key="synthetic"))
            if r == R - 1:
                tasks.append(TaskSpec(f"opt_{i}", (f"W_{i}", f"dW_{i}", f"O_{i}"), (), mutates=(f"W_{i}", f"O_{i}"), runtime_us=c["opt_us"],
                                      compute_block_key="synthetic"))
    final = {f"W_{i}": "backing" for i in range(L)} | {f"O_{i}": "backing" for i in range(L)}
    return Program(name="engine_gate", initial_objects=tuple(init), tasks=tuple(tasks), final_locations=final,
                   bandwidth_from_slow=52000, bandwidth_to_slow=52000)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", default="mini", choices=sorted(CONFIGS))
    ap.add_argument("--fast-gib", type=float, required=True)
    ap.add_argument("--backend", default="cpu", choices=["fake", "cpu", "cuda"])
    ap.add_argument("--completion-mode", default="poll", choices=["poll", "hostfn"])
    ap.add_argument("--repeat", type=int, default=3)
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    from dataflow_b200.lowering.planning import plan_program
    from dataflow_b200.runtime import CpuBackend, Engine, FakeBackend, Session, synthetic_resolver, trace_to_dict
    prog = synthetic_program(CONFIGS[a.config])
    planned = plan_program(prog, int(a.fast_gib * (1 << 30)), leeway_bytes=0)
    if a.backend == "cuda":
        from dataflow_b200.runtime import CudaBackend
        be = CudaBackend(0, a.completion_mode)
        from dataflow_b200.run.driver import HostStore
        sizes = {o.id: o.size_bytes for o in planned.program.initial_objects}
        store = HostStore(be, sizes, pinned=True)
        initial = store.buffers()
    else:
        be = FakeBackend() if a.backend == "fake" else CpuBackend()
        store, initial = None, None
    eng = Engine(be, session=Session(be))
    best = None
    for _ in range(a.repeat):
        res = eng.execute(planned.program, synthetic_resolver, initial, dispatch_ahead=2 if a.backend == "cuda" else 0)
        res.raise_if_failed()
        if best is None or res.makespan_us < best.makespan_us:
            best = res
    ratio = best.makespan_us / planned.makespan_us
    summary = {"config": a.config, "backend": a.backend, "tasks": len(prog.tasks), "sim_ms": planned.makespan_us / 1e3,
               "real_ms": best.makespan_us / 1e3, "gap_pct": 100.0 * (ratio - 1.0), "sim_peak_bytes": planned.peak_fast_bytes,
               "real_peak_bytes": best.peak_fast_bytes, "peak_equal": best.peak_fast_bytes == planned.peak_fast_bytes,
               "dispatch_us_per_task": best.stats.get("dispatch_us_total", 0.0) / len(prog.tasks), "policy": planned.policy}
    print(json.dumps(summary, indent=1))
    if a.out:
        os.makedirs(a.out, exist_ok=True)
        stem = os.path.join(a.out, f"engine_gate-{a.config}")
        json.dump(summary, open(stem + ".summary.json", "w"), indent=1)
        json.dump(trace_to_dict(best.trace), open(stem + ".trace.json", "w"))
    if store is not None:
        store.close()
    return 0 if summary["peak_equal"] or a.backend == "cuda" else 1


if __name__ == "__main__":
    raise SystemExit(main())
