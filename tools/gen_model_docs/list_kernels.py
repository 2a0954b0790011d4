"""List every registered op with its implementations (eager / library / sm100), which one resolves on this machine, and
whether it is native code.

    python tools/gen_model_docs/list_kernels.py [--kernel-set eager]

Reference role: ``tools/gen_model_docs/list_kernels.py``.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from _cli import table  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--kernel-set", default=None)
    a = ap.parse_args(argv)
    from dataflow_b200.ops import registered_ops, resolve_kernels
    ks = resolve_kernels(kernel_set=a.kernel_set)
    chosen = ks.describe()
    rows = [{"op": op, "implementations": ", ".join(sorted(k.name for k in impls)), "resolved": chosen.get(op, "-"),
             "native": "yes" if op in ks.native_ops() else ""} for op, impls in sorted(registered_ops().items())]
    print(table(rows, [("op", "{}"), ("implementations", "{}"), ("resolved", "{}"), ("native", "{}")]))
    print(f"{len(rows)} ops; {len(ks.native_ops())} resolve to native code here")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
