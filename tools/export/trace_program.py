"""Plan debugging without a GPU: run ANY program on the virtual-time backend and print its event timeline — reserves,
transfer enqueues and completions, releases, offloads, pressure evictions, placement escapes.

    python tools/export/trace_program.py --program examples/llama3-tiny.annotated.json --kinds offload,prefetch --intervals

Reference role: ``tools/export/trace_program.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import _cli  # noqa: E402,F401


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--program", required=True)
    ap.add_argument("--kinds", default=None, help="comma list: only events whose kind contains one of these")
    ap.add_argument("--intervals", action="store_true")
    ap.add_argument("--out", default=None, help="write events as JSONL instead of a table")
    a = ap.parse_args(argv)
    from dataflow_b200.core.jsonio import load_program
    from dataflow_b200.runtime import Engine, FakeBackend, synthetic_resolver
    prog = load_program(a.program)
    res = Engine(FakeBackend()).execute(prog, synthetic_resolver, record_events=True)
    kinds = a.kinds.split(",") if a.kinds else None
    events = [e for e in res.trace.events if kinds is None or any(k in e.kind for k in kinds)]
    if a.out:
        with open(a.out, "w") as f:
            for e in events:
                f.write(json.dumps({"kind": e.kind, "what": e.what, "fast_bytes": e.fast_bytes}) + "\n")
    else:
        for e in events:
            print(f"{e.kind:<22} {e.what:<40} fast {e.fast_bytes}")
    if a.intervals:
        for iv in sorted(res.trace.intervals, key=lambda i: (i.start_us, i.track)):
            print(f"{iv.start_us:12.2f} .. {iv.end_us:12.2f}  {iv.track:<10} {iv.name}")
    print(f"outcome {res.outcome.kind.value}; makespan {res.makespan_us:.2f} us; peak fast {res.peak_fast_bytes} B; "
          f"pressure evictions {res.stats.get('pressure_evictions', 0)}, placement escapes {res.stats.get('placement_escapes', 0)}")
    return 0 if res.outcome.ok else 1


if __name__ == "__main__":
    raise SystemExit(main())
