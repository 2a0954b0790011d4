"""What every stage shares: where results live, how a finished stage is kept on ``--resume``, small statistics."""
from __future__ import annotations

import json
import math
import os
import time


def stage(out: str, name: str, resume: bool, fn):
    """Run ``fn`` and write its value to ``<out>/<name>.json``; with ``resume`` a file that exists is read back instead."""
    path = os.path.join(out, name + ".json")
    if resume and os.path.exists(path):
        print(f"[{name}] kept {path}")
        with open(path) as f:
            return json.load(f)
    t0 = time.time()
    val = fn()
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        json.dump(val, f, indent=1)
    os.replace(tmp, path)                      # a stage killed half-way leaves no file that --resume would trust
    print(f"[{name}] done in {time.time() - t0:.1f}s -> {path}")
    return val


def geomean(xs) -> float:
    xs = [x for x in xs if x and x > 0]
    return math.exp(sum(math.log(x) for x in xs) / len(xs)) if xs else float("nan")


def quantile(xs, q: float) -> float:
    xs = sorted(xs)
    if not xs:
        return float("nan")
    pos = q * (len(xs) - 1)
    lo, hi = int(math.floor(pos)), int(math.ceil(pos))
    return xs[lo] + (xs[hi] - xs[lo]) * (pos - lo)


def append_jsonl(path: str, row: dict) -> None:
    with open(path, "a") as f:
        f.write(json.dumps(row) + "\n")
        f.flush()
        os.fsync(f.fileno())


def read_jsonl(path: str) -> list[dict]:
    if not os.path.exists(path):
        return []
    rows = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line:
                try:
                    rows.append(json.loads(line))
                except ValueError:
                    pass                         # a line cut short by a kill: the cell is measured again
    return rows
