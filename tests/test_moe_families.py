"""MoE families (olmoe, qwen3moe) and qwen3: engine vs pure-torch twin from identical init and data."""
import dataclasses

import pytest
import torch

from dataflow_b200.models.families import resolve_family, validate_family
from dataflow_b200.run.driver import Trainer, synthetic_rounds


def run_pair(family, device, policy, steps=3, budget=None, **over):
    fam = resolve_family(family)
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy=policy, **over)
    hyper = {"lr": 2e-3, "weight_decay": 0.1}
    tr = Trainer(family, cfg, budget_gib=budget, device=device, hyper=hyper, seed=3, leeway_bytes=0)
    try:
        twin = fam.twin(cfg)
        twin.load_state_dict(fam.bridge(cfg, tr.views_of))
        decay = [p for _, p in twin.named_parameters() if p.dim() >= 2]
        plain = [p for _, p in twin.named_parameters() if p.dim() < 2]
        opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": plain, "weight_decay": 0.0}], lr=2e-3,
                                betas=(0.9, 0.95), eps=1e-8)
        bounds = list(range(0, tr.T + 1, cfg.seq_len))
        eng, ref = [], []
        for s in range(steps):
            data = synthetic_rounds(cfg, tr.rounds, tr.T, 64, 11, s)
            opt.zero_grad()
            tot = 0.0
            for tk, tg in data:
                l = twin.loss(tk, tg, bounds, total_rows=tr.T * tr.rounds)
                l.backward()
                tot += float(l.detach())
            opt.step()
            ref.append(tot)
            eng.append(tr.step(data))
    finally:
        tr.close()
    return eng, ref


@pytest.mark.parametrize("family", ["qwen3", "olmoe", "qwen3moe"])
def test_family_structure(family):
    assert validate_family(family) == []


@pytest.mark.parametrize("family", ["qwen3", "olmoe", "qwen3moe"])
def test_cpu_fp32_engine_matches_twin(family):
    eng, ref = run_pair(family, None, "fp32")
    assert eng[0] == pytest.approx(ref[0], rel=1e-4)
    for a, b in zip(eng, ref):
        assert a == pytest.approx(b, rel=5e-4)
    assert eng[-1] < eng[0]


def test_moe_recompute_levels_are_invisible_in_the_losses():
    a, _ = run_pair("olmoe", None, "fp32", steps=2, budget=None)
    b, _ = run_pair("olmoe", None, "fp32", steps=2, budget=0.03)
    assert a == pytest.approx(b, rel=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("family", ["olmoe", "qwen3moe"])
def test_gpu_moe_engine_in_band(family):
    eng, ref = run_pair(family, 0, "bf16_split_master")
    for a, b in zip(eng, ref):
        assert a == pytest.approx(b, rel=4e-2)
    assert eng[-1] < eng[0]
