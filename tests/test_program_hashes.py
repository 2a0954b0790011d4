"""Lowered-program content hashes, pinned.

Refactors of the lowering, the layouts or the planner must not change WHAT a family lowers to: same tasks, same compute
keys, same block parameters, same byte sizes, same order.  This gate pins the sha256 of the canonical JSON of every
family's ``tiny`` preset — bare (what the family's lowering says), planned with room to spare, and planned under pressure
(70 % of the roomy plan's peak, where the planner has to offload, prefetch or recompute; the planner is deterministic) —
against a committed fixture.  Regenerate ONLY when a content change is intended:

    DATAFLOW_REGEN_HASHES=1 python -m pytest tests/test_program_hashes.py

Parity: reference ``tests/test_program_hashes.py``.
"""
import hashlib
import json
import os
from pathlib import Path

import pytest

FIXTURE = Path(__file__).parent / "fixtures" / "program_hashes.json"
PLAN_BUDGET = 1 << 30


def program_hash(program) -> str:
    from dataflow_b200.core.jsonio import program_to_dict
    blob = json.dumps(program_to_dict(program), sort_keys=True, separators=(",", ":"))
    return hashlib.sha256(blob.encode()).hexdigest()


def current_hashes() -> dict:
    from dataflow_b200.lowering import resolve_hardware
    from dataflow_b200.lowering.planning import PlanningError
    from dataflow_b200.models.families import _BUILTIN, all_families
    from dataflow_b200.run.driver import plan_at_budget
    hw = resolve_hardware("b200")            # a fixed hardware row: the hashes must not depend on the machine
    out = {}
    for name, fam in sorted(all_families().items()):
        if "tiny" not in fam.presets or name not in _BUILTIN:        # plugins registered by other tests are not pinned
            continue
        cfg = fam.presets["tiny"]()
        bare = fam.lower(cfg, hw=hw)
        roomy = plan_at_budget(fam, cfg, PLAN_BUDGET, hw, leeway_bytes=0)
        try:
            tight = program_hash(plan_at_budget(fam, cfg, roomy.max_workspace + int(0.7 * roomy.peak_fast_bytes), hw, leeway_bytes=0).program)
        except PlanningError:
            tight = "infeasible"
        out[name] = {"bare": program_hash(bare), "planned": program_hash(roomy.program), "tight": tight, "tasks": len(bare.tasks)}
    return out


def test_lowered_program_hashes_stable():
    now = current_hashes()
    if os.environ.get("DATAFLOW_REGEN_HASHES"):
        FIXTURE.write_text(json.dumps(now, indent=1, sort_keys=True) + "\n")
    pinned = json.loads(FIXTURE.read_text())
    assert sorted(now) == sorted(pinned), "a family appeared or disappeared: regenerate the fixture if that is intended"
    drift = {k: (pinned[k], v) for k, v in now.items() if pinned[k] != v}
    assert not drift, f"lowered programs changed for {sorted(drift)}; regenerate the fixture if that is intended"


def test_lowering_is_repeatable_within_a_process():
    from dataflow_b200.lowering import resolve_hardware
    from dataflow_b200.models.families import resolve_family
    fam = resolve_family("llama3")
    hw = resolve_hardware("b200")
    a, b = fam.lower(fam.presets["tiny"](), hw=hw), fam.lower(fam.presets["tiny"](), hw=hw)
    assert program_hash(a) == program_hash(b)
