"""Deep correctness compare, one family x shape: ONE optimizer step of the engine against the pure-torch twin from
identical weights and data, judged in dW space.

    python tools/verify/deep_compare.py --family llama3 --shape ragged --hot-mult 1.5

Per parameter tensor it reports the relative L2 distance of the weight updates, and classifies every element whose
update differs: AdamW's first step moves an element by about +-lr according to the SIGN of its gradient, so an element
whose gradient is within rounding noise of zero may legitimately go the other way (a *near-tie flip*); an element
with a solid gradient that goes the other way is a real disagreement.  The gate: no real flips, and the update
distance over the non-tie elements below ``--tol``.  Activations between tasks and saved contexts are bf16 under every
dtype policy, so the engine's gradients carry bf16 rounding noise that the fp32 twin's do not: "within noise of zero"
means below ``--tie-rel`` of the local gradient scale, and a handful of real flips per million elements is allowed
(``--real-ppm``).  Reference role: ``tools/verify/deep_compare.py``.
"""
from __future__ import annotations

import argparse
import dataclasses
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from _cli import table  # noqa: E402


def deep_compare(family: str, shape: str = "uniform", hot_mult: float = 1.0, device=None, policy: str = "fp32",
                 tie_rel: float = 0.3, seed: int = 3):
    import torch
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    from dataflow_b200.testing.family_gate import ragged_bounds
    fam = resolve_family(family)
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy=policy)
    hyper = {"lr": 2e-3, "weight_decay": 0.1}
    tr = Trainer(family, cfg, budget_gib=None, device=device, hyper=hyper, seed=seed, leeway_bytes=0)
    rows = []
    try:
        if hot_mult != 1.0:
            for oid in tr.store.sizes:
                if oid.startswith("W_"):
                    for v in tr.views_of(oid, tr.layouts.layout_of(oid)).values():
                        if v.dim() >= 2:
                            v.mul_(hot_mult)
        w0 = {k: v.clone().float() for k, v in fam.bridge(cfg, tr.views_of).items()}
        twin = fam.twin(cfg)
        twin.load_state_dict(fam.bridge(cfg, tr.views_of))
        decay = [p for _, p in twin.named_parameters() if p.dim() >= 2]
        plain = [p for _, p in twin.named_parameters() if p.dim() < 2]
        opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": plain, "weight_decay": 0.0}], lr=2e-3,
                                betas=(0.9, 0.95), eps=1e-8)
        data = synthetic_rounds(cfg, tr.rounds, tr.T, 64, 11, 0)
        bounds = {r: (ragged_bounds(tr.T, cfg.seq_len, r) if shape == "ragged" else list(range(0, tr.T + 1, cfg.seq_len)))
                  for r in range(tr.rounds)}
        opt.zero_grad()
        ref_loss = 0.0
        for r, (tk, tg) in enumerate(data):
            l = twin.loss(tk, tg, bounds[r], total_rows=tr.T * tr.rounds)
            l.backward()
            ref_loss += float(l.detach())
        grads = {n: p.grad.detach().float().clone() for n, p in twin.named_parameters() if p.grad is not None}
        opt.step()
        eng_loss = tr.step(data, seq_lens=bounds if shape == "ragged" else None)
        tr.sync_to_host()
        mine, theirs = fam.bridge(cfg, tr.views_of), twin.state_dict()
        for k in sorted(w0):
            if k not in theirs or k not in grads:
                continue
            dm, dt, g = mine[k].float() - w0[k], theirs[k].float() - w0[k], grads[k]
            differ = (dm - dt).abs() > 0.5 * hyper["lr"]
            tie = g.abs() < tie_rel * _local_scale(g)
            real = differ & ~tie
            solid = ~tie
            d_solid = float((dm - dt)[solid].norm() / (dt[solid].norm() + 1e-30)) if solid.any() else 0.0
            rows.append({"tensor": k, "dW_rel_l2": float((dm - dt).norm() / (dt.norm() + 1e-30)), "dW_rel_l2_solid": d_solid,
                         "flips": int(differ.sum()), "near_tie": int((differ & tie).sum()), "real": int(real.sum()), "n": dm.numel()})
    finally:
        tr.close()
    return {"family": family, "shape": shape, "loss_engine": eng_loss, "loss_twin": ref_loss, "rows": rows}


def _local_scale(g):
    """Typical gradient magnitude around every element: the median of the non-zero |g| of its column and of its row
    (the smaller of the two; different heads and unused vocabulary rows have very different scales)."""
    import torch
    a = g.abs()
    if a.dim() == 3:                      # stacked experts: every expert has its own scale
        return torch.stack([_local_scale(x) for x in g])
    if a.dim() < 2:
        nz = a[a > 0]
        return torch.full_like(a, float(nz.median()) if nz.numel() else 0.0) + 1e-30
    def med(dim):
        x = torch.where(a > 0, a, torch.full_like(a, float("nan")))
        return torch.nan_to_num(x.nanmedian(dim=dim, keepdim=True).values, nan=0.0)
    return torch.minimum(med(0).expand_as(a), med(1).expand_as(a)) + 1e-30


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--family", required=True)
    ap.add_argument("--shape", default="uniform", choices=["uniform", "ragged"])
    ap.add_argument("--hot-mult", type=float, default=1.0)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--policy", default="fp32")
    ap.add_argument("--tol", type=float, default=3e-2)
    ap.add_argument("--tie-rel", type=float, default=0.3)
    ap.add_argument("--real-ppm", type=float, default=100.0)
    a = ap.parse_args(argv)
    out = deep_compare(a.family, a.shape, a.hot_mult, None if a.device == "cpu" else int(a.device), a.policy, a.tie_rel)
    print(f"{a.family} / {a.shape}: loss engine {out['loss_engine']:.6f} twin {out['loss_twin']:.6f}")
    print(table(out["rows"], [("tensor", "{}"), ("n", "{}"), ("dW_rel_l2", "{:.2e}"), ("dW_rel_l2_solid", "{:.2e}"), ("flips", "{}"),
                              ("near_tie", "{}"), ("real", "{}")]))
    bad = [r for r in out["rows"] if r["real"] * 1e6 > a.real_ppm * r["n"] or r["dW_rel_l2_solid"] > a.tol]
    print("PASS" if not bad else f"FAIL: {[r['tensor'] for r in bad]}")
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
