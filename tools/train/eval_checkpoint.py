"""Evaluate a checkpoint: load it into the family's pure-torch twin (through the same bridge the parity gates use) and
report the mean token loss and perplexity over held-out data.

    python tools/train/eval_checkpoint.py --checkpoint ckpt/step_000100 --preset llama3:tiny --data 'shards:data/mine,split=val' --steps 20

Only the weights are read, so checkpoints of solo, replica (``co``) and sharded (``fsdp`` / ``zero*``) runs of any world size
evaluate alike; tensor- and expert-parallel checkpoints hold per-rank cuts of the model and are not assembled here.

Reference role: ``tools/train/eval_checkpoint.py``.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import _cli  # noqa: E402,F401


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--checkpoint", required=True, help="a step directory written by train.py")
    ap.add_argument("--preset", required=True)
    ap.add_argument("--data", default=None, help="data spec (default: seeded synthetic documents)")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args(argv)
    import torch
    from dataflow_b200.data.pipeline import pipeline_from_args
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.run.checkpointing import load_checkpoint, peek
    from dataflow_b200.run.driver import Trainer
    from dataflow_b200.run.presets import resolve_preset
    fam_name, cfg = resolve_preset(a.preset)
    fam = resolve_family(fam_name)
    # the run's own overrides of the preset (dtype policy, layers, sequence length, ...) are in the checkpoint's launch record
    import dataclasses
    from dataflow_b200.checkpoint.record import read_record
    resolved = dict(((read_record(a.checkpoint).get("launch") or {}).get("resolved")) or {})
    known = {f.name for f in dataclasses.fields(cfg)}
    over = {k: v for k, v in resolved.items() if k in known and k not in ("name", "tp", "ep", "grad_accum_rounds")}
    if over:
        cfg = dataclasses.replace(cfg, **over)
    tr = Trainer(fam_name, cfg, budget_gib=None, device=None, init=True)
    info = load_checkpoint(tr, a.checkpoint, only_prefixes=("W_",))       # weights alone: any data-parallel sharding restores
    twin = fam.twin(cfg)
    twin.load_state_dict(fam.bridge(cfg, tr.views_of))
    dev = torch.device("cpu" if a.device == "cpu" else f"cuda:{a.device}")
    twin.to(dev)
    stepper = pipeline_from_args(cfg, a.data)()
    total, rows = 0.0, 0
    with torch.no_grad():
        for _ in range(a.steps):
            step = stepper.next_step()
            if step is None:
                break
            for r in step.rounds:
                tk, tg = torch.as_tensor(r.tokens).to(dev), torch.as_tensor(r.targets).to(dev)
                valid = int((tg >= 0).sum())
                if not valid:
                    continue
                bounds = list(r.bounds) + ([len(r.tokens)] if r.bounds[-1] < len(r.tokens) else [])
                total += float(twin.loss(tk, tg, bounds, total_rows=1))
                rows += valid
    stepper.close()
    tr.close()
    mean = total / max(rows, 1)
    out = {"checkpoint": peek(a.checkpoint)["step"], "tokens": rows, "loss": mean, "perplexity": math.exp(min(mean, 50.0)), "resumed": info.get("step")}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
