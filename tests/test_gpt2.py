"""gpt2 family: engine vs twin (tied and untied, fp32 on the CPU backend) and the 124M fp32
plumbing configuration planned at a 2 GiB fast budget and stepped once on the host."""
import dataclasses
import time

import pytest
import torch

from dataflow_b200.models.families import resolve_family, validate_family
from dataflow_b200.run.driver import Trainer, synthetic_rounds


def twin_losses(fam, cfg, tr, data, hyper):
    twin = fam.twin(cfg)
    twin.load_state_dict(fam.bridge(cfg, tr.views_of))
    decay = [p for p in twin.parameters() if p.dim() >= 2]
    plain = [p for p in twin.parameters() if p.dim() < 2]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": hyper["weight_decay"]}, {"params": plain, "weight_decay": 0.0}],
                            lr=hyper["lr"], betas=(0.9, 0.95), eps=1e-8)
    bounds = list(range(0, tr.T + 1, cfg.seq_len))
    out = []
    for step in data:
        opt.zero_grad()
        tot = 0.0
        for tk, tg in step:
            l = twin.loss(tk, tg, bounds, total_rows=tr.T * tr.rounds)
            l.backward()
            tot += float(l.detach())
        opt.step()
        out.append(tot)
    return out


def test_structure():
    assert validate_family("gpt2") == []


@pytest.mark.parametrize("tied", [False, True])
def test_engine_matches_twin_fp32(tied):
    fam = resolve_family("gpt2")
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32", act_dtype="fp32", tied_embeddings=tied)
    hyper = {"lr": 1e-3, "weight_decay": 0.1}
    tr = Trainer("gpt2", cfg, budget_gib=None, device=None, hyper=hyper, seed=1)
    data = [synthetic_rounds(cfg, tr.rounds, tr.T, 64, 3, s) for s in range(3)]
    ref = twin_losses(fam, cfg, tr, data, hyper)
    eng = [tr.step(d) for d in data]
    tr.close()
    for a, b in zip(eng, ref):
        assert a == pytest.approx(b, rel=1e-5)
    assert eng[-1] < eng[0]


def test_gpt2_124m_fp32_one_step_on_cpu_planned_at_2gib():
    """GPT-2 124M, fp32, seq 1024, batch 2, 2 accumulation rounds, AdamW 6e-4, tied, vocab 50257."""
    fam = resolve_family("gpt2")
    cfg = fam.presets["gpt2_124m_fp32"]()
    torch.manual_seed(0)
    tr = Trainer("gpt2", cfg, budget_gib=2.0, device=None, hyper={"lr": 6e-4, "weight_decay": 0.1}, seed=0,
                 leeway_bytes=64 << 20)
    assert tr.planned.budget == 2 << 30
    assert tr.planned.peak_fast_bytes + tr.planned.max_workspace <= 2 << 30
    assert tr.program.is_annotated() and tr.planned.transfer["from_slow"]["count"] > 0       # it really streams
    g = torch.Generator().manual_seed(0)
    data = []
    for _ in range(tr.rounds):
        ids = torch.randint(0, 50257, (tr.T + 1,), generator=g)
        data.append((ids[:-1].int(), ids[1:].int()))
    t0 = time.time()
    loss = tr.step(data)
    res = tr.last_result
    tr.close()
    assert 10.0 < loss < 11.6                     # ln(50257) = 10.82 at init
    assert res.peak_fast_bytes <= tr.planned.object_capacity
    print(f"gpt2-124m fp32 CPU step: loss {loss:.4f} in {time.time() - t0:.1f}s, peak fast {res.peak_fast_bytes / 2**20:.0f} MiB")
