"""Kernel-time shares of one real step: which kernels the compute lane spends its time in, per launch and in total.

    python tools/bench/kernel_shares.py --preset llama3_8b --layers 4 --ga-rounds 2          # a cut of the model, no budget
    python tools/bench/kernel_shares.py --preset olmoe:tiny --top 20

Runs two warm-up steps, then one step under the torch profiler (CUDA activities only) and prints, per kernel name, the
launch count, the mean and the total device time and its share.  The times are taken under a profiler: read them as
SHARES and per-launch comparisons between kernels, never as benchmark numbers.  Copies on the host link appear as
``Memcpy`` rows; they run on their own streams beside the compute lane.
"""
from __future__ import annotations

import argparse
import collections
import dataclasses
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import _cli  # noqa: E402,F401


def kernel_shares(trainer, data) -> tuple[float, list[tuple[str, int, float]]]:
    """(total device µs, [(kernel name, launches, total µs)] sorted by time) of one step of ``trainer`` on ``data``."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        trainer.step(data)
        torch.cuda.synchronize()
    agg: dict[str, list[float]] = collections.defaultdict(lambda: [0, 0.0])
    for e in prof.events():
        if e.device_type == torch.autograd.DeviceType.CUDA:
            agg[e.name][0] += 1
            agg[e.name][1] += e.device_time
    rows = sorted(((k, int(v[0]), float(v[1])) for k, v in agg.items()), key=lambda r: -r[2])
    return sum(r[2] for r in rows), rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="llama3_8b", help="preset name or family:preset")
    ap.add_argument("--layers", type=int, default=None, help="cut the model to this many layers")
    ap.add_argument("--ga-rounds", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--dtype-policy", default=None)
    ap.add_argument("--budget", type=float, default=None, help="device budget GiB (default: unbounded)")
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--top", type=int, default=40)
    a = ap.parse_args(argv)
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    from dataflow_b200.run.presets import resolve_preset
    fam, cfg = resolve_preset(a.preset)
    over = {k: v for k, v in (("n_layers", a.layers), ("grad_accum_rounds", a.ga_rounds), ("seq_len", a.seq_len), ("batch", a.batch),
                              ("dtype_policy", a.dtype_policy)) if v is not None}
    cfg = dataclasses.replace(cfg, **over)
    tr = Trainer(fam, cfg, budget_gib=a.budget, device=a.device, hyper={"lr": 3e-4, "weight_decay": 0.1}, seed=0, profile=False,
                 lower_kwargs={"resident_params": True})
    try:
        vocab = getattr(cfg, "vocab_size", 1024)
        for s in range(2):
            tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, vocab, 0, s, pin=True))
        total, rows = kernel_shares(tr, synthetic_rounds(cfg, tr.rounds, tr.T, vocab, 0, 2, pin=True))
    finally:
        tr.close()
    print(f"total device time {total / 1e3:.1f} ms over {len(rows)} kernels; layer-rounds: {cfg.n_layers * tr.rounds}")
    for name, n, us in rows[:a.top]:
        print(f"{us / 1e3:9.2f} ms {100 * us / total:5.1f}%  n={n:5d}  avg {us / n:9.1f} us  {name[:110]}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
