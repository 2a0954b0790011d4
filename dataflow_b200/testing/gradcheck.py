"""Gradient checks of a family's engine lowering against autograd through its pure-torch twin.

The engine never exposes gradients (they are consumed by the optimizer tasks that follow the last backward), so the
check reads them off a plain SGD step: with learning rate 1, no momentum and no weight decay the update is
``w <- w - g``, hence ``g = w_before - w_after`` per parameter tensor.  The twin's gradients come from ``loss.backward()``
on the same data and the same initial bytes.

``check_model_step``     every parameter tensor of the model (embedding, every layer, head)
``check_block_backward`` a one-layer cut of the model, reporting the block's own fields — the backward of one block
                         against autograd, with the (already checked) embedding and head around it

Reference role: ``src/dataflow_training/testing/gradcheck.py`` (``check_block_backward`` :132, ``reference_model_step`` :223,
``check_model_step`` :629, ``rel_l2``, ``CheckReport``).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Any, Mapping


def rel_l2(a, b) -> float:
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


@dataclass
class CheckReport:
    family: str
    loss_engine: float
    loss_twin: float
    grad_rel_l2: dict[str, float] = field(default_factory=dict)
    grad_norm: dict[str, float] = field(default_factory=dict)
    tol: float = 2e-2
    loss_tol: float = 1e-4

    @property
    def loss_rel(self) -> float:
        return abs(self.loss_engine - self.loss_twin) / max(abs(self.loss_twin), 1e-12)

    def failures(self) -> dict[str, float]:
        # a tensor whose gradient is (numerically) zero on both sides has no direction to compare
        return {k: v for k, v in self.grad_rel_l2.items() if v > self.tol and self.grad_norm[k] > 1e-10}

    def __bool__(self) -> bool:
        return self.loss_rel <= self.loss_tol and not self.failures()

    def summary(self) -> str:
        worst = sorted(self.grad_rel_l2.items(), key=lambda kv: -kv[1])[:5]
        return (f"{self.family}: loss {self.loss_engine:.6f} vs twin {self.loss_twin:.6f} (rel {self.loss_rel:.2e}); "
                f"{len(self.grad_rel_l2)} tensors, worst " + ", ".join(f"{k} {v:.2e}" for k, v in worst))


def check_model_step(family: str, *, preset: str = "tiny", overrides: Mapping[str, Any] | None = None, device: int | None = None,
                     policy: str = "fp32", shape: str = "uniform", seed: int = 3, tol: float = 2e-2, budget_gib: float | None = None,
                     only_prefix: str | None = None, kernels=None) -> CheckReport:
    """One optimizer step of the engine lowering against one ``loss.backward()`` of the twin; gradients compared per tensor.

    ``tol``: activations and saved context are bf16 under every dtype policy (the policy governs parameters, gradients
    and optimizer state), while the twin computes in fp32 throughout: dense families agree to about 0.5 % per tensor.
    Mixture-of-experts families need a looser bound (0.25): a token whose two best router scores nearly tie may be
    routed differently by the two sides, which moves a few rows between experts (with ``top_k = n_experts`` in
    ``overrides`` nothing can flip and the same families agree to about 1 %).  A wrong backward is off by O(1)."""
    import torch
    from ..models.families import resolve_family
    from ..run.driver import Trainer, synthetic_rounds
    from .family_gate import ragged_bounds
    fam = resolve_family(family)
    cfg = dataclasses.replace(fam.presets[preset](), dtype_policy=policy, optimizer="sgd", **dict(overrides or {}))
    hyper = {"optimizer": "sgd", "lr": 1.0, "weight_decay": 0.0, "momentum": 0.0, "schedule": {"kind": "constant", "peak_lr": 1.0}}
    tr = Trainer(family, cfg, budget_gib=budget_gib, device=device, hyper=hyper, seed=seed, leeway_bytes=0, kernels=kernels)
    try:
        before = fam.bridge(cfg, tr.views_of)
        twin = fam.twin(cfg)
        twin.load_state_dict(before)
        data = synthetic_rounds(cfg, tr.rounds, tr.T, 64, 11, 0)
        if shape == "ragged":
            bounds = {r: ragged_bounds(tr.T, cfg.seq_len, r) for r in range(tr.rounds)}
        else:
            bounds = {r: list(range(0, tr.T + 1, cfg.seq_len)) for r in range(tr.rounds)}
        twin.zero_grad()
        loss_twin = 0.0
        for r, (tk, tg) in enumerate(data):
            loss = twin.loss(tk, tg, bounds[r], total_rows=tr.T * tr.rounds)
            loss.backward()
            loss_twin += float(loss.detach())
        loss_engine = tr.step(data, seq_lens=bounds if shape == "ragged" else None)
        tr.sync_to_host()
        after = fam.bridge(cfg, tr.views_of)
    finally:
        tr.close()
    rep = CheckReport(family, float(loss_engine), loss_twin, tol=tol)
    grads = {k: p.grad for k, p in twin.named_parameters()}
    for k, w0 in before.items():
        if k not in grads or (only_prefix and not k.startswith(only_prefix)):
            continue
        g_ref = grads[k] if grads[k] is not None else torch.zeros_like(w0)
        g_eng = w0.float() - after[k].float()
        rep.grad_rel_l2[k] = rel_l2(g_eng, g_ref)
        rep.grad_norm[k] = float(g_ref.float().norm())
    return rep


def check_block_backward(family: str, *, kind_layer: int = 0, **kw) -> CheckReport:
    """The backward of ONE block against autograd: a cut of the model that ends right after layer ``kind_layer`` (so the
    layer kinds before it keep their place in families that mix kinds), reporting that layer's fields only."""
    over = dict(kw.pop("overrides", None) or {})
    over["n_layers"] = int(kind_layer) + 1
    return check_model_step(family, overrides=over, only_prefix=f"layers.{int(kind_layer)}.", **kw)
