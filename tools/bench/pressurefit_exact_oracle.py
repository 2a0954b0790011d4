"""Exact oracle for tiny chains: enumerate EVERY placement of offload / prefetch / release directives a planner could
emit on a chain of a few tasks, keep the feasible ones, and compare the best makespan with each policy's.

    python tools/bench/pressurefit_exact_oracle.py --chains 20 --tasks 4 --seed 0

``--policies`` takes any names of the planner registry (default: pressurefit, lookahead).  A policy that is more than
``--tolerance`` worse than the oracle on any chain is reported and the exit code is 1.  On 6-task chains PressureFit finds
the optimum, Lookahead, max_reduce and min_grow stay within about 1 % of it, roundtrip within 10 %; the reactive planner
(no placement up front, fetches as late as it can) pays up to 20 %, the fixed window pattern up to 45 %.
The search is exponential: keep ``--tasks`` at 5 or below.  Reference role: ``tools/bench/pressurefit_exact_oracle.py``.
"""
from __future__ import annotations

import argparse
import itertools
import os
import random
import sys
from dataclasses import replace

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import _cli  # noqa: E402,F401


def random_chain(rng: random.Random, n_tasks: int):
    """Forward / backward shaped chain: weights start in host memory, activations are made by the forward half and
    consumed in reverse by the backward half."""
    from dataflow_b200.sim.schema import Object, OutputAlloc, Task, TaskChain
    half = max(n_tasks // 2, 1)
    unit = 1000
    init = [Object(f"w{i}", unit * rng.randint(1, 4), "backing", "parameter") for i in range(half)]
    tasks = []
    for i in range(half):
        tasks.append(Task(f"f{i}", [f"w{i}"] + ([f"x{i}"] if i else []),
                          [OutputAlloc(f"a{i}", unit * rng.randint(1, 4), "fast", "activation"), OutputAlloc(f"x{i + 1}", unit, "fast", "activation")],
                          float(rng.randint(5, 20))))
    for i in reversed(range(half)):
        tasks.append(Task(f"b{i}", [f"w{i}", f"a{i}", f"x{i + 1}" if i == half - 1 else f"g{i + 1}"],
                          [OutputAlloc(f"g{i}", unit, "fast", "activation")], float(rng.randint(5, 20))))
    sizes = {o.id: o.size for o in init}
    need = max(sum(sizes.get(i, 4 * unit) for i in t.inputs) + sum(o.size for o in t.outputs) for t in tasks)
    return TaskChain(init, tasks, {f"w{i}": "backing" for i in range(half)}, fast_memory_capacity=int(need * 1.3),
                     bandwidth_from_slow=400, bandwidth_to_slow=400)


def oracle_makespan(chain, limit: int = 200000) -> tuple[float, int]:
    """Best makespan over all directive placements (weights prefetched after some task before their use; every
    activation optionally offloaded after its producer and prefetched back before its consumer)."""
    from dataflow_b200.sim.schema import TransferTrigger
    from dataflow_b200.sim.simulator import run as simulate
    tasks = chain.tasks
    idx = {t.id: i for i, t in enumerate(tasks)}
    uses: dict[str, list[int]] = {}
    for i, t in enumerate(tasks):
        for o in t.inputs:
            uses.setdefault(o, []).append(i)
    producer = {o.id: i for i, t in enumerate(tasks) for o in t.outputs}
    choices = []        # per object: list of (offload_after task | None, [prefetch_after task per later use | None])
    objs = sorted(uses)
    for o in objs:
        us = uses[o]
        opts = []
        if o in producer:                                            # activation: stay, or round-trip before its last use
            opts.append(("stay", None, None))
            last = us[-1]
            for off in range(producer[o], last - 1):
                for pre in range(off, last):
                    opts.append(("trip", off, pre))
        else:                                                        # weight: start on the device, or when to bring it in
            # (between two uses it may also be dropped and fetched again: ``a`` = the task after which it comes back)
            again = [None] + (list(range(us[0], us[-1])) if len(us) > 1 else [])
            for back in again:
                opts.append(("resident", back, None))
                for pre in range(0, us[0]):
                    opts.append(("in", back, pre))
        choices.append(opts)
    best, tried = float("inf"), 0
    for combo in itertools.product(*choices):
        tried += 1
        if tried > limit:
            break
        off = {i: [] for i in range(len(tasks))}
        pre = {i: [] for i in range(-1, len(tasks))}
        rel = {i: [] for i in range(len(tasks))}
        resident = {o for o, (kind, _, _) in zip(objs, combo) if kind == "resident"}
        for o, (kind, a, b) in zip(objs, combo):
            if kind == "trip":
                off[a].append(TransferTrigger(o))
                pre[b].append(TransferTrigger(o))
            else:
                if kind == "in":
                    pre[b].append(TransferTrigger(o))
                if a is not None:                            # dropped after its first use, back after task ``a``
                    rel[uses[o][0]].append(o)
                    pre[a].append(TransferTrigger(o))
            rel[uses[o][-1]].append(o)
        new = [replace(t, offload_after=off[i], prefetch_after=pre[i], releases_after=rel[i]) for i, t in enumerate(tasks)]
        try:
            # a resident weight has a device copy beside its host copy from the start
            init = list(chain.initial_memory) + [replace(o, location="fast") for o in chain.initial_memory if o.id in resident]
            m = simulate(replace(chain, tasks=new, initial_memory=init), validate=False).makespan
        except Exception:
            continue
        best = min(best, m)
    return best, tried


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--chains", type=int, default=10)
    ap.add_argument("--tasks", type=int, default=4)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--policies", default="pressurefit,lookahead")
    ap.add_argument("--tolerance", type=float, default=0.10)
    a = ap.parse_args(argv)
    from dataflow_b200.sim.policies import get_all_policies
    from dataflow_b200.sim.simulator import run as simulate
    rng = random.Random(a.seed)
    pols = {k: v for k, v in get_all_policies().items() if k in a.policies.split(",")}
    worst = {k: 0.0 for k in pols}
    bad = 0
    for c in range(a.chains):
        chain = random_chain(rng, a.tasks)
        best, tried = oracle_makespan(chain)
        line = f"chain {c}: oracle {best:.1f} us over {tried} placements;"
        for name, fn in pols.items():
            try:
                m = simulate(fn(chain, chain.fast_memory_capacity), validate=False).makespan
            except Exception as e:
                line += f" {name} FAILED ({type(e).__name__})"
                bad += 1
                continue
            excess = m / best - 1.0 if best < float("inf") else 0.0
            worst[name] = max(worst[name], excess)
            line += f" {name} {m:.1f} ({excess:+.1%})"
            if excess > a.tolerance:
                bad += 1
        print(line)
    print("worst excess over the oracle: " + ", ".join(f"{k} {v:+.1%}" for k, v in worst.items()))
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
