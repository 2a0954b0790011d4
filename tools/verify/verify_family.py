"""One-command family correctness: structure check (lowering validates, every compute key resolves, layouts agree with
object sizes), the engine-versus-twin model step on uniform and ragged shapes, per-tensor gradients against autograd
through the twin, plan invariance under a tight budget, and an audit that the family has its canonical tests in ``tests/``.

    python tools/verify/verify_family.py --family olmoe
    python tools/verify/verify_family.py --list
    python tools/verify/verify_family.py --family llama3 --audit-only

Reference role: ``tools/verify/verify_family.py``.
"""
from __future__ import annotations

import argparse
import glob
import os
import re
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import _cli  # noqa: E402,F401

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
CANON = {"structure": r"validate_family|test_(family_)?structure", "twin step": r"twin", "plan invariance / budget": r"budget|invariance|recompute"}


def audit(family: str) -> list[str]:
    """Which canonical checks no test file mentions for this family."""
    texts = [open(p).read() for p in glob.glob(os.path.join(ROOT, "tests", "test_*.py"))]
    mine = [t for t in texts if re.search(rf"['\"]{re.escape(family)}['\"]", t)]
    if not mine:
        return [f"no test module mentions family {family!r}"]
    return [f"no test covers: {name}" for name, pat in CANON.items() if not any(re.search(pat, t) for t in mine)]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--family", default=None)
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--audit-only", action="store_true")
    ap.add_argument("--plugin", action="append", default=[])
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--tol", type=float, default=1e-3)
    a = ap.parse_args(argv)
    import importlib
    for m in a.plugin:
        importlib.import_module(m)
    from dataflow_b200.models.families import all_families, validate_family
    if a.list:
        for name, fam in sorted(all_families().items()):
            print(f"{name:<12} presets: {', '.join(sorted(fam.presets))}")
        return 0
    if not a.family:
        ap.error("--family or --list")
    problems = audit(a.family)
    for p in problems:
        print("audit:", p)
    if a.audit_only:
        return 1 if problems else 0
    bad = list(problems)
    issues = validate_family(a.family)
    print("structure:", "ok" if not issues else issues)
    bad += issues
    from dataflow_b200.testing.family_gate import run_pair
    device = None if a.device == "cpu" else int(a.device)
    base = None
    for shape in ("uniform", "ragged"):
        r = run_pair(a.family, device=device, policy="fp32" if device is None else "bf16_master", shape=shape)
        ok = r["max_loss_rel"] < (a.tol if device is None else 3e-2) and r["engine"][-1] < r["engine"][0]
        print(f"model step / {shape:<8}: max loss rel {r['max_loss_rel']:.2e}, curve {r['engine'][0]:.4f} -> {r['engine'][-1]:.4f}  {'ok' if ok else 'FAIL'}")
        if not ok:
            bad.append(f"model step {shape}")
        if shape == "uniform":
            base = r["engine"]
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.testing.gradcheck import check_model_step
    cfg0 = resolve_family(a.family).presets["tiny"]()
    routed = bool(getattr(cfg0, "n_experts", 0) or getattr(cfg0, "moe", False))
    rep = check_model_step(a.family, device=device, policy="fp32" if device is None else "bf16_master",
                           tol=(0.25 if routed else 2e-2) if device is None else 0.35)
    print(f"gradients   : {rep.summary()}  {'ok' if rep else 'FAIL'}")
    if not rep:
        bad.append(f"gradients {sorted(rep.failures())[:4]}")
    tight = run_pair(a.family, device=device, policy="fp32" if device is None else "bf16_master", budget_gib=0.03)
    same = max(abs(x - y) / abs(y) for x, y in zip(tight["engine"], base)) < 1e-5
    print(f"plan invariance at 0.03 GiB: {'ok' if same else 'FAIL'}")
    if not same:
        bad.append("plan invariance")
    print("PASS" if not bad else f"FAIL: {bad}")
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
