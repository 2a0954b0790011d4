"""One-command family correctness, as a ladder of rungs that each print one line:

    audit            the family has its canonical tests in ``tests/``
    structure        the lowering validates, every compute key resolves, layouts agree with object sizes
    model step       engine against twin over a few optimizer steps, uniform and ragged shapes
    gradients        every parameter tensor's gradient against autograd through the twin (relative L2 and cosine)
    block backward   the same for one layer of every block kind the family mixes
    recompute        a backward that rebuilds its context gives the gradients of one that saved it
    accumulation     a step of two rounds gives the sum of its rounds run alone
    plan invariance  a tight device budget changes the plan, not the loss curve
    client           (``--through-daemon``) the gradients rung through a daemon client, from fetched host copies

``--rungs a,b`` runs a subset.

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
    ap.add_argument("--rungs", default=None, help="comma list of: structure, step, gradients, block, recompute, accumulation, invariance, client")
    ap.add_argument("--through-daemon", action="store_true", help="add the client rung (a daemon in this process, CPU backend)")
    a = ap.parse_args(argv)
    rungs = ("structure", "step", "gradients", "block", "recompute", "accumulation", "invariance", "client")
    want = {r.strip() for r in a.rungs.split(",") if r.strip()} if a.rungs else set(rungs[:-1])
    if want - set(rungs):
        ap.error(f"--rungs {','.join(sorted(want - set(rungs)))}: no such rung (known: {', '.join(rungs)})")
    if a.through_daemon:
        want.add("client")
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
    if a.family not in all_families():
        ap.error(f"--family {a.family}: unknown model family (known: {', '.join(sorted(all_families()))}; --plugin MODULE registers more)")
    problems = audit(a.family)
    for p in problems:
        print("audit:", p)
    if a.audit_only:
        return 1 if problems else 0
    bad = list(problems)
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.testing import gradcheck
    from dataflow_b200.testing.family_gate import run_pair
    device = None if a.device == "cpu" else int(a.device)
    policy = "fp32" if device is None else "bf16_master"
    fam = resolve_family(a.family)
    cfg0 = fam.presets["tiny"]()
    routed = bool(getattr(cfg0, "n_experts", 0) or getattr(cfg0, "moe", False))
    gtol = (0.25 if routed else 2e-2) if device is None else 0.35

    def rung(name, fn):
        """Run one rung; an exception is a failure of that rung, not of the tool."""
        try:
            ok, line = fn()
        except Exception as e:     # noqa: BLE001
            ok, line = False, f"{type(e).__name__}: {str(e)[:200]}"
        print(f"{name:<16}: {line}  {'ok' if ok else 'FAIL'}")
        if not ok:
            bad.append(name)

    if "structure" in want:
        issues = validate_family(a.family)
        rung("structure", lambda: (not issues, "validates" if not issues else str(issues)))
    base = None
    if "step" in want or "invariance" in want:
        for shape in ("uniform", "ragged") if "step" in want else ("uniform",):
            r = run_pair(a.family, device=device, policy=policy, shape=shape)
            if shape == "uniform":
                base = r["engine"]
            if "step" in want:
                rung(f"step / {shape}", lambda r=r: (r["max_loss_rel"] < (a.tol if device is None else 3e-2) and r["engine"][-1] < r["engine"][0],
                                                     f"max loss rel {r['max_loss_rel']:.2e}, curve {r['engine'][0]:.4f} -> {r['engine'][-1]:.4f}, "
                                                     f"weights within {r['max_weight_rel_l2']:.1e}"))
    if "gradients" in want:
        def grads():
            rep = gradcheck.check_model_step(a.family, device=device, policy=policy, tol=gtol)
            return bool(rep), rep.summary() + (f"; failing {sorted(rep.failures())[:4]}" if not rep else "")
        rung("gradients", grads)
    if "block" in want:
        # the kind of every layer, read off the lowered program: the compute key of its forward task in the first round
        fwd = sorted(((int(t.id.rsplit("_", 1)[1]), t.compute_block_key) for t in fam.lower(cfg0).tasks if t.id.startswith("block_fwd_0_0_")))
        kinds = [k for _, k in fwd]
        layers = sorted({kinds.index(k) for k in set(kinds)}) if kinds else [0]       # the first layer of every kind
        for i in layers:
            def block(i=i):
                rep = gradcheck.check_block_backward(a.family, device=device, policy=policy, tol=gtol, kind_layer=i)
                what = f"layer {i}" + (f" ({kinds[i]})" if kinds else "")
                return bool(rep), (f"{what}: {len(rep.grad_rel_l2)} tensors, worst {max(rep.grad_rel_l2.values(), default=0.0):.2e}, "
                                   f"lowest cosine {min(rep.grad_cos.values(), default=1.0):.5f}")
            rung("block backward", block)
    if "recompute" in want:
        def recompute():
            d = gradcheck.check_recompute_equivalence(a.family, device=device, policy=policy, tol=1e-5 if device is None else 2e-2)
            if not d:
                return True, "the family's backward rebuilds its context itself (no recompute tasks, no levels): nothing to compare"
            return True, f"{len(d)} tensors, largest distance between rebuilt and saved contexts {max(d.values(), default=0.0):.1e}"
        rung("recompute", recompute)
    if "accumulation" in want:
        def accumulation():
            d = gradcheck.check_accumulation(a.family, device=device, policy=policy, tol=5e-4 if device is None else 5e-2)
            return True, f"{len(d)} tensors, largest distance between a 2-round step and the sum of its rounds {max(d.values(), default=0.0):.1e}"
        rung("accumulation", accumulation)
    if "invariance" in want and base is not None:
        def invariance():
            tight = run_pair(a.family, device=device, policy=policy, budget_gib=0.03)
            d = max(abs(x - y) / abs(y) for x, y in zip(tight["engine"], base))
            return d < (1e-5 if device is None else 3e-2), f"0.03 GiB against unconstrained: max rel. distance of the curves {d:.1e}"
        rung("plan invariance", invariance)
    if "client" in want:
        def client():
            from dataflow_b200.testing.client_parity import client_model_step
            from dataflow_b200.testing.server_process import engine_client
            with engine_client(backing_gib=0.5, device=None) as c:
                rep = client_model_step(c, a.family, tol=0.25 if routed else 2e-2)
            return bool(rep), rep.summary()
        rung("client", client)
    print("PASS" if not bad else f"FAIL: {bad}")
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
