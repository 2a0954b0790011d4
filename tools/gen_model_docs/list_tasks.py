"""List the tasks of a preset's lowered program: compute key, inputs, outputs, cost seed, workspace.

    python tools/gen_model_docs/list_tasks.py --preset olmoe:tiny [--round 0]

Reference role: ``tools/gen_model_docs/list_tasks.py``.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from _cli import table  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--preset", default="llama3:tiny")
    ap.add_argument("--round", type=int, default=None)
    a = ap.parse_args(argv)
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.run.presets import resolve_preset
    fam, cfg = resolve_preset(a.preset)
    prog = resolve_family(fam).lower(cfg)
    rows = []
    for t in prog.tasks:
        if a.round is not None and t.block_params.get("round", a.round) != a.round:
            continue
        rows.append({"task": t.id, "key": t.compute_block_key, "inputs": " ".join(t.inputs), "outputs": " ".join(o.id for o in t.outputs),
                     "mutates": " ".join(t.mutates), "us": t.runtime_us, "ws_kib": t.workspace_bytes / 1024})
    print(table(rows, [("task", "{}"), ("key", "{}"), ("us", "{:.1f}"), ("ws_kib", "{:.0f}"), ("inputs", "{}"), ("outputs", "{}"), ("mutates", "{}")]))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
