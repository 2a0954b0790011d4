"""Gradient checks of a family's engine lowering against autograd through its pure-torch twin.

The engine never exposes gradients (they are consumed by the optimizer tasks that follow the last backward), so the
check reads them off a plain SGD step: with learning rate 1, no momentum and no weight decay the update is
``w <- w - g``, hence ``g = w_before - w_after`` per parameter tensor.  The twin's gradients come from ``loss.backward()``
on the same data and the same initial bytes.

``check_model_step``     every parameter tensor of the model (embedding, every layer, head)
``check_block_backward`` a one-layer cut of the model, reporting the block's own fields — the backward of one block
                         against autograd, with the (already checked) embedding and head around it
``check_recompute_equivalence``  the same step with contexts rebuilt before the backward and with contexts saved: equal gradients
``check_accumulation``   a step of several rounds against the sum of its rounds run alone

Every per-tensor comparison reports a relative L2 distance (size) and a cosine (direction).

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


def cos_sim(a, b) -> float:
    """Cosine of the angle between two tensors taken as flat fp64 vectors: the direction check beside ``rel_l2``'s size
    check.  Two zero vectors agree (1.0); a zero vector against a non-zero one does not (0.0)."""
    a, b = a.detach().double().reshape(-1), b.detach().double().reshape(-1)
    na, nb = float(a.norm()), float(b.norm())
    if na == 0.0 and nb == 0.0:
        return 1.0
    if na == 0.0 or nb == 0.0:
        return 0.0
    return float(a @ b) / (na * nb)


@dataclass
class CheckReport:
    family: str
    loss_engine: float
    loss_twin: float
    grad_rel_l2: dict[str, float] = field(default_factory=dict)
    grad_norm: dict[str, float] = field(default_factory=dict)
    grad_cos: dict[str, float] = field(default_factory=dict)
    engine_gradients: dict[str, Any] = field(default_factory=dict)      # filled on request (``keep_gradients``)
    weight_norm: dict[str, float] = field(default_factory=dict)
    recompute_tasks: int = 0
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
        low = min(self.grad_cos.values(), default=1.0)
        return (f"{self.family}: loss {self.loss_engine:.6f} vs twin {self.loss_twin:.6f} (rel {self.loss_rel:.2e}); "
                f"{len(self.grad_rel_l2)} tensors, lowest cosine {low:.5f}, worst " + ", ".join(f"{k} {v:.2e}" for k, v in worst))


def check_model_step(family: str, *, preset: str = "tiny", overrides: Mapping[str, Any] | None = None, device: int | None = None,
                     policy: str = "fp32", shape: str = "uniform", seed: int = 3, tol: float = 2e-2, budget_gib: float | None = None,
                     only_prefix: str | None = None, kernels=None, lower_kwargs: Mapping[str, Any] | None = None,
                     keep_gradients: bool = False, round_of: tuple[int, int] | None = None) -> CheckReport:
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
    tr = Trainer(family, cfg, budget_gib=budget_gib, device=device, hyper=hyper, seed=seed, leeway_bytes=0, kernels=kernels,
                 lower_kwargs=lower_kwargs, recompute=lower_kwargs is None)
    try:
        before = fam.bridge(cfg, tr.views_of)
        twin = fam.twin(cfg)
        twin.load_state_dict(before)
        data = synthetic_rounds(cfg, tr.rounds, tr.T, 64, 11, 0)
        rows_of_step = tr.T * tr.rounds
        if round_of is not None:            # this one-round step is round ``r`` of a step of ``n`` rounds: same tokens, same normalisation
            r_, n_ = round_of
            if tr.rounds != 1:
                raise ValueError("round_of needs a one-round configuration")
            data = [synthetic_rounds(cfg, n_, tr.T, 64, 11, 0)[r_]]
            rows_of_step = tr.T * n_
        if shape == "ragged":
            bounds = {r: ragged_bounds(tr.T, cfg.seq_len, r) for r in range(tr.rounds)}
        else:
            bounds = {r: list(range(0, tr.T + 1, cfg.seq_len)) for r in range(tr.rounds)}
        twin.zero_grad()
        loss_twin = 0.0
        for r, (tk, tg) in enumerate(data):
            loss = twin.loss(tk, tg, bounds[r], total_rows=rows_of_step)
            loss.backward()
            loss_twin += float(loss.detach())
        loss_engine = tr.step(data, seq_lens=bounds if shape == "ragged" else None, valid_rows=rows_of_step)
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
        rep.grad_cos[k] = cos_sim(g_eng, g_ref)
        rep.grad_norm[k] = float(g_ref.float().norm())
        rep.weight_norm[k] = float(w0.float().norm())
        if keep_gradients:
            rep.engine_gradients[k] = g_eng.clone()
    rep.recompute_tasks = sum(1 for t in tr.program.tasks if "recompute" in t.id)
    return rep


READ_EPS = 1.2e-7    # a gradient read as w_before - w_after carries an absolute error of up to about this much x |w| (fp32 rounding)


def _rel_beyond_rounding(a, b, weight_norm: float, reads: int = 2) -> float:
    """Relative L2 distance of two gradients that were both read off weight differences, after taking off what rounding
    of the reads alone can explain (``reads`` x READ_EPS x |w|): a tensor whose gradient is tiny beside its weights (a norm
    gain near 1 with a gradient near 1e-5) is not reported for rounding, and a real difference still is."""
    a, b = a.float(), b.float()
    return max(float((a - b).norm()) - reads * READ_EPS * weight_norm, 0.0) / (float(b.norm()) + 1e-30)


def check_recompute_equivalence(family: str, *, level: int = 2, layers=None, tol: float = 1e-5, **kw) -> dict[str, float]:
    """A backward that rebuilds its context must give the gradients of one that saved it.  Runs the same step twice, once
    with every layer (or ``layers``) lowered at recompute ``level`` and once with everything saved, and returns the
    relative L2 distance of the engine's gradients per tensor; raises ``AssertionError`` naming the tensors above ``tol``.
    (The two runs execute the same kernels on the same bytes in the same order within a block, so on one device they
    agree to rounding of the few ops whose inputs take another path: well under 1e-5 in fp32.)"""
    from ..models.families import resolve_family
    fam = resolve_family(family)
    cfg = fam.presets[kw.get("preset", "tiny")]()
    n_layers = int(dict(kw.get("overrides") or {}).get("n_layers", fam.derive_dims(cfg).n_layers))
    which = list(range(n_layers)) if layers is None else list(layers)
    if not which:
        raise AssertionError("the lowering did not honour the levels: no layer was asked to recompute")
    saved = check_model_step(family, keep_gradients=True, lower_kwargs={"recompute_levels": {}}, **kw)
    rebuilt = check_model_step(family, keep_gradients=True, lower_kwargs={"recompute_levels": {i: level for i in which}}, **kw)
    if rebuilt.recompute_tasks == 0 and saved.recompute_tasks == 0 and not fam.lower(cfg).recompute_rewrites:
        # a family whose backward keeps nothing but the block input and rebuilds the rest itself has no separate recompute
        # tasks and offers no levels: there are no two forms to compare
        return {}
    if rebuilt.recompute_tasks == 0 or saved.recompute_tasks != 0:
        raise AssertionError(f"the lowering did not honour the levels: {saved.recompute_tasks} recompute tasks without, "
                             f"{rebuilt.recompute_tasks} with")
    dist = {k: _rel_beyond_rounding(rebuilt.engine_gradients[k], g, saved.weight_norm.get(k, 0.0), 2) for k, g in saved.engine_gradients.items()
            if float(g.float().norm()) > 1e-10}
    bad = {k: v for k, v in dist.items() if v > tol}
    if bad or abs(saved.loss_engine - rebuilt.loss_engine) > tol * max(abs(saved.loss_engine), 1.0):
        raise AssertionError(f"{family}: recomputed and saved contexts disagree: loss {saved.loss_engine} vs {rebuilt.loss_engine}, "
                             f"tensors {sorted(bad.items(), key=lambda kv: -kv[1])[:5]}")
    return dist


def check_accumulation(family: str, *, rounds: int = 2, tol: float = 5e-4, **kw) -> dict[str, float]:
    """Gradients accumulate: a step of ``rounds`` rounds gives the sum of the gradients its rounds give alone.  The rounds
    alone are run as single-round steps over the same token blocks with the loss normalised by the rows of the WHOLE step,
    so the sums are comparable; returns the per-tensor relative L2 distance.  Gradients are read as weight differences,
    which costs an absolute error of up to about 1.2e-7 x |w| per read in fp32; that much (once per step compared) is
    taken off the distance first, so tensors with tiny gradients beside large weights are not reported for rounding.  A step that
    dropped or doubled a round is off by O(1)."""
    import torch
    over = dict(kw.pop("overrides", None) or {})
    whole = check_model_step(family, keep_gradients=True, overrides={**over, "grad_accum_rounds": rounds}, **kw)
    total: dict[str, Any] = {}
    for r in range(rounds):
        part = check_model_step(family, keep_gradients=True, overrides={**over, "grad_accum_rounds": 1}, **kw, round_of=(r, rounds))
        for k, g in part.engine_gradients.items():
            total[k] = g if k not in total else total[k] + g
    dist = {k: _rel_beyond_rounding(total[k], g, whole.weight_norm.get(k, 0.0), rounds + 1) for k, g in whole.engine_gradients.items()
            if float(g.float().norm()) > 1e-10}
    bad = {k: v for k, v in dist.items() if v > tol}
    if bad:
        raise AssertionError(f"{family}: a {rounds}-round step is not the sum of its rounds: {sorted(bad.items(), key=lambda kv: -kv[1])[:5]}")
    return dist


def check_block_backward(family: str, *, kind_layer: int = 0, **kw) -> CheckReport:
    """The backward of ONE block against autograd: a cut of the model that ends right after layer ``kind_layer`` (so the
    layer kinds before it keep their place in families that mix kinds), reporting that layer's fields only."""
    over = dict(kw.pop("overrides", None) or {})
    over["n_layers"] = int(kind_layer) + 1
    return check_model_step(family, overrides=over, only_prefix=f"layers.{int(kind_layer)}.", **kw)
