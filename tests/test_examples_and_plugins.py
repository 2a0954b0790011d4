"""The RL example (program surgery on a family's lowering) and a family registered from outside the package."""
import dataclasses
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_rl_program_surgery():
    from dataflow_b200.core.validate import validate_program
    from dataflow_b200.models.families import resolve_family
    from examples.rl_training.builder import build_rl_program
    cfg = resolve_family("llama3").presets["tiny"]()
    prog = build_rl_program("llama3", cfg)
    validate_program(prog)
    keys = [t.compute_block_key for t in prog.tasks]
    assert "head_loss" not in keys and keys.count("rl_head_loss") == cfg.grad_accum_rounds
    assert keys.count("block_recompute") == cfg.n_layers * cfg.grad_accum_rounds            # one in front of every backward
    head = next(t for t in prog.tasks if t.compute_block_key == "rl_head_loss")
    assert any(i.startswith("advantages_") for i in head.inputs) and any(i.startswith("old_logprobs_") for i in head.inputs)
    assert not any(o.startswith("A_") for t in prog.tasks if t.compute_block_key == "block_fwd" for o in (x.id for x in t.outputs))


@pytest.mark.parametrize("objective", ["ppo", "reinforce"])
def test_policy_loss_gradient_matches_autograd(objective):
    from examples.rl_training.rl_ops import policy_loss_fwd_bwd
    torch.manual_seed(0)
    logits = torch.randn(40, 17)
    actions = torch.randint(0, 17, (40,), dtype=torch.int32)
    actions[::7] = -1
    adv, old = torch.randn(40), torch.log_softmax(torch.randn(40, 17), -1).gather(1, actions.clamp(min=0).long()[:, None])[:, 0]
    z = logits.clone().requires_grad_(True)
    lp = torch.log_softmax(z, -1).gather(1, actions.clamp(min=0).long()[:, None])[:, 0]
    if objective == "ppo":
        r = torch.exp(lp - old)
        per = -torch.minimum(r * adv, r.clamp(0.8, 1.2) * adv)
    else:
        per = -adv * lp
    ref = (per * (actions >= 0).float()).sum() / 33.0
    ref.backward()
    out = torch.zeros(1)
    work = logits.clone()
    policy_loss_fwd_bwd(work, actions, adv, old, 33.0, out, objective=objective)
    assert out.item() == pytest.approx(ref.item(), rel=1e-5)
    assert torch.allclose(work, z.grad, atol=1e-6)


def test_rl_harness_raises_the_reward():
    from examples.rl_training.harness import RLTrainer
    from dataflow_b200.models.families import resolve_family
    cfg = dataclasses.replace(resolve_family("llama3").presets["tiny"](), dtype_policy="fp32")
    rl = RLTrainer("llama3", cfg, device=None, objective="ppo", lr=5e-3)
    gen = torch.Generator().manual_seed(0)
    tr, small = rl.tr, 16
    bounds = list(range(0, tr.T + 1, cfg.seq_len))
    means = []
    try:
        for s in range(7):
            rounds, rewards = [], []
            for r in range(tr.rounds):
                tk = torch.randint(0, small, (tr.T,), generator=gen, dtype=torch.int32)
                act, lp = rl.rollout(tk, bounds, gen)
                reward = (act == (tk + 1) % small).float()
                rewards.append(float(reward.mean()))
                rounds.append((tk, act, reward - reward.mean(), lp))
            rl.step(rounds)
            means.append(sum(rewards) / len(rewards))
    finally:
        rl.close()
    assert means[-1] > 10 * max(means[0], 1.0 / cfg.vocab_size)


def test_external_family_registers_validates_and_trains():
    import importlib
    importlib.import_module("tests.fixtures.external_family.toy_family")
    from dataflow_b200.models.families import all_families, validate_family
    from dataflow_b200.testing.family_gate import run_pair
    assert "toy" in all_families() and validate_family("toy") == []
    r = run_pair("toy", steps=3)
    assert r["max_loss_rel"] < 1e-3 and r["engine"][-1] < r["engine"][0]


def test_plugin_flag_of_the_tools_loads_an_external_family():
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tools", "bench", "predict_step.py"), "--plugin",
                        "tests.fixtures.external_family.toy_family", "--preset", "toy:tiny", "--budget", "1"],
                       capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "tok_s" in r.stdout and "INFEASIBLE" not in r.stdout
