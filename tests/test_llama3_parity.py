"""Engine vs pure-torch twin from byte-identical init and data (the correctness gate)."""
import dataclasses

import pytest
import torch

from dataflow_b200.models.families import resolve_family, validate_family
from dataflow_b200.run.driver import Trainer, synthetic_rounds


def twin_curve(cfg, tr, data_steps, hyper, steps):
    fam = resolve_family("llama3")
    twin = fam.twin(cfg)
    twin.load_state_dict(fam.bridge(cfg, tr.views_of))
    decay = [p for n, p in twin.named_parameters() if p.dim() >= 2]
    plain = [p for n, p in twin.named_parameters() if p.dim() < 2]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": hyper.get("weight_decay", 0.0)},
                             {"params": plain, "weight_decay": 0.0}], lr=hyper["lr"], betas=(0.9, 0.95), eps=1e-8)
    bounds = list(range(0, tr.T + 1, cfg.seq_len))
    losses = []
    for s in range(steps):
        opt.zero_grad()
        total = 0.0
        for tk, tg in data_steps[s]:
            l = twin.loss(tk, tg, bounds, total_rows=tr.T * tr.rounds)
            l.backward()
            total += float(l.detach())
        opt.step()
        losses.append(total)
    return losses


def run_pair(device, policy, steps=4, budget=None, lower_kwargs=None):
    fam = resolve_family("llama3")
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy=policy)
    hyper = {"lr": 2e-3, "weight_decay": 0.1}
    tr = Trainer("llama3", cfg, budget_gib=budget, device=device, hyper=hyper, seed=3, leeway_bytes=0,
                 lower_kwargs=lower_kwargs)
    try:
        data = [synthetic_rounds(cfg, tr.rounds, tr.T, 64, 11, s) for s in range(steps)]   # small id range: learnable
        ref = twin_curve(cfg, tr, data, hyper, steps)
        eng = [tr.step(data[s]) for s in range(steps)]
    finally:
        tr.close()
    return eng, ref


def test_family_structure():
    assert validate_family("llama3") == []


def test_cpu_fp32_engine_matches_twin_tightly():
    eng, ref = run_pair(None, "fp32")
    assert eng[0] == pytest.approx(ref[0], rel=1e-5)
    for a, b in zip(eng, ref):
        assert a == pytest.approx(b, rel=2e-4)
    assert eng[-1] < eng[0]


def test_cpu_bf16_engine_in_band():
    eng, ref = run_pair(None, "bf16_master")
    for a, b in zip(eng, ref):
        assert a == pytest.approx(b, rel=3e-2)


def test_plan_invariance_on_cpu():
    """The same math under a tight budget (offload / prefetch / recompute) gives the same losses."""
    a, _ = run_pair(None, "fp32", steps=3, budget=None)
    b, _ = run_pair(None, "fp32", steps=3, budget=0.02)
    assert a == pytest.approx(b, rel=1e-6)


def test_split_master_policy_tracks_fp32_master_policy():
    """Same fp32 master either way; only the moments differ (bf16 vs fp32 storage)."""
    a, ref = run_pair(None, "bf16_split_master")
    b, _ = run_pair(None, "bf16_master")
    for x, y in zip(a, b):
        assert x == pytest.approx(y, rel=5e-3)
    assert a[-1] < a[0]


@pytest.mark.parametrize("budget", [None, 0.02])
def test_resident_params_give_the_same_losses(budget):
    """Weights that stay on the fast tier between steps (never re-read from the host store) train identically."""
    a, _ = run_pair(None, "fp32", steps=4, budget=budget)
    b, _ = run_pair(None, "fp32", steps=4, budget=budget, lower_kwargs={"resident_params": True})
    assert a == pytest.approx(b, rel=1e-6)


@pytest.mark.gpu
def test_gpu_split_master_resident_in_band():
    eng, ref = run_pair(0, "bf16_split_master", lower_kwargs={"resident_params": True})
    for a, b in zip(eng, ref):
        assert a == pytest.approx(b, rel=3e-2)
    assert eng[-1] < eng[0]


@pytest.mark.gpu
def test_gpu_engine_in_band_and_native():
    eng, ref = run_pair(0, "bf16_master")
    for a, b in zip(eng, ref):
        assert a == pytest.approx(b, rel=3e-2)
    assert eng[-1] < eng[0]


@pytest.mark.gpu
def test_gpu_plan_invariance():
    a, _ = run_pair(0, "bf16", steps=3, budget=None)
    b, _ = run_pair(0, "bf16", steps=3, budget=0.02)
    assert a == pytest.approx(b, rel=1e-3)
