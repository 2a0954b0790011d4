"""Reference arm of the benchmark: runs the unmodified reference (installed under
``baseline/_ref``) through its own public API on the same metric and config.
Prints ``{"impl": "reference", "unavailable": ...}`` when it cannot run here."""
from __future__ import annotations

import os
import sys


def run_reference_arm(a) -> dict:
    rank = int(os.environ.get("RANK", 0))
    ref = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
    if not os.path.isdir(os.path.join(ref, "dataflow_training")):
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed on this machine"} if rank == 0 else {}
    return {"impl": "reference", "unavailable": "reference arm not wired yet"} if rank == 0 else {}
