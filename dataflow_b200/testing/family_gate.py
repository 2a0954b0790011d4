"""Engine-versus-twin gates shared by the verification tools and the family tests.

``run_pair`` trains a family's engine lowering and its pure-torch twin from byte-identical initial weights on the
same data and returns both loss curves plus, per parameter tensor, the relative L2 distance of the final weights.
Ragged shapes (several sequences of different lengths packed into a round) exercise the varlen paths.
Reference role: the ladder-3 "model step" gate of ``tests/dataflow_training/model_families/*`` and
``src/dataflow_training/testing/client_parity.py``.
"""
from __future__ import annotations

import dataclasses
from typing import Any


def ragged_bounds(tokens: int, seq_len: int, seed: int = 0) -> list[int]:
    """Cumulative sequence boundaries [0, b1, ..., tokens] with uneven lengths no longer than ``seq_len``."""
    import random
    rng = random.Random(seed)
    out, at = [0], 0
    while at < tokens:
        n = min(rng.randint(max(seq_len // 4, 1), seq_len), tokens - at)
        at += n
        out.append(at)
    return out


def run_pair(family: str, *, device: int | None = None, policy: str = "fp32", steps: int = 3, budget_gib: float | None = None,
             shape: str = "uniform", hot_mult: float = 1.0, seed: int = 3, hyper: dict | None = None,
             preset: str = "tiny", overrides: dict | None = None) -> dict[str, Any]:
    import torch
    from ..models.families import resolve_family
    from ..run.driver import Trainer, synthetic_rounds
    fam = resolve_family(family)
    cfg = dataclasses.replace(fam.presets[preset](), dtype_policy=policy, **dict(overrides or {}))
    hyper = dict(hyper or {"lr": 2e-3, "weight_decay": 0.1})
    tr = Trainer(family, cfg, budget_gib=budget_gib, device=device, hyper=hyper, seed=seed, leeway_bytes=0)
    try:
        if hot_mult != 1.0:                                  # larger weights make gradient differences visible
            for oid in tr.store.sizes:
                if oid.startswith("W_"):
                    for v in tr.views_of(oid, tr.layouts.layout_of(oid)).values():
                        if v.dim() >= 2:
                            v.mul_(hot_mult)
        twin = fam.twin(cfg)
        twin.load_state_dict(fam.bridge(cfg, tr.views_of))
        import fnmatch
        only = tuple(getattr(cfg, "trainable_patterns", ()) or ())          # runs that update a named subset of fields
        live = [(n, p) for n, p in twin.named_parameters()
                if not only or any(fnmatch.fnmatchcase(n.rsplit(".", 1)[-1], pat) for pat in only)]
        decay = [p for _, p in live if p.dim() >= 2]
        plain = [p for _, p in live if p.dim() < 2]
        opt = torch.optim.AdamW([{"params": decay, "weight_decay": hyper.get("weight_decay", 0.0)},
                                 {"params": plain, "weight_decay": 0.0}], lr=hyper["lr"], betas=(0.9, 0.95), eps=1e-8)
        eng, ref = [], []
        for s in range(steps):
            data = synthetic_rounds(cfg, tr.rounds, tr.T, 64, 11, s)
            if shape == "ragged":
                bounds = {r: ragged_bounds(tr.T, cfg.seq_len, 100 * s + r) for r in range(tr.rounds)}
            else:
                bounds = {r: list(range(0, tr.T + 1, cfg.seq_len)) for r in range(tr.rounds)}
            opt.zero_grad()
            tot = 0.0
            for r, (tk, tg) in enumerate(data):
                loss = twin.loss(tk, tg, bounds[r], total_rows=tr.T * tr.rounds)
                loss.backward()
                tot += float(loss.detach())
            opt.step()
            ref.append(tot)
            eng.append(tr.step(data, seq_lens=bounds if shape == "ragged" else None))
        tr.sync_to_host()
        mine = fam.bridge(cfg, tr.views_of)
        theirs = twin.state_dict()
        dist = {}
        for k, v in mine.items():
            if k in theirs:
                a, b = v.float(), theirs[k].float()
                dist[k] = float((a - b).norm() / (b.norm() + 1e-12))
    finally:
        tr.close()
    return {"family": family, "shape": shape, "policy": policy, "engine": eng, "twin": ref, "weight_rel_l2": dist,
            "max_weight_rel_l2": max(dist.values()) if dist else 0.0,
            "max_loss_rel": max(abs(a - b) / max(abs(b), 1e-12) for a, b in zip(eng, ref))}
