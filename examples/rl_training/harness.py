"""A small RL loop on the engine: sample actions from the current policy (the twin computes the rollout log-probabilities
from the engine's weights), score them with a reward, and take policy-gradient steps through the RL program.

    python examples/rl_training/harness.py --family llama3 --steps 6 --objective ppo

The toy task: the reward of a token is 1 when the sampled next token equals (token + 1) mod vocab_small.  The mean
reward rises within a few steps.  Reference role: ``examples/rl_training/harness.py:83-315``.
"""
from __future__ import annotations

import argparse
import dataclasses
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from examples.rl_training.builder import build_rl_program  # noqa: E402
from examples.rl_training.rl_ops import policy_loss_fwd_bwd  # noqa: E402


def make_rl_head(base_cls):
    """``RLHeadLoss``: the family's head executable with the policy-gradient loss in place of cross-entropy."""

    class RLHeadLoss(base_cls):
        objective = "ppo"
        clip_eps = 0.2

        def run(self, ctx):
            import torch
            d, K = self.dims, self.K
            n = self.segments(ctx).n_tokens
            y = self.tview(ctx.inputs[0], (d.T, d.d))[:n]
            act = self.tview(ctx.inputs[1], (d.T,), "int32")[:n]
            w = self.views(ctx.inputs[2], self.lay.head_w)
            adv = self.tview(self.by_id(ctx, "advantages_"), (d.T,), "fp32")[:n]
            old = self.tview(self.by_id(ctx, "old_logprobs_"), (d.T,), "fp32")[:n]
            dy = self.tview(ctx.outputs[0], (d.T, d.d))[:n]
            loss = self.tview(ctx.outputs[1], (1,), "fp32")
            create = self.creating(ctx, "dW_head")
            dw = self.views(self.by_id(ctx, "dW_head"), self.lay.head_dw)
            total_rows = float(ctx.run_args.get("valid_rows", n))
            loss_dev = torch.zeros(1, dtype=torch.float32, device=y.device)
            first = True
            for lo in range(0, n, d.head_chunk):
                hi = min(lo + d.head_chunk, n)
                yc = y[lo:hi]
                xn, rstd = K.rmsnorm_fwd(yc, w["final_norm"], d.eps)
                logits = K.linear_fwd_bf16(xn, w["w_head"])
                policy_loss_fwd_bwd(logits, act[lo:hi], adv[lo:hi].to(logits.device), old[lo:hi].to(logits.device), total_rows, loss_dev,
                                    objective=self.objective, clip_eps=self.clip_eps, accumulate=not first)
                acc = not (create and first)
                K.linear_wgrad_bf16(xn, logits, dw["w_head"], accumulate=acc)
                dxn = K.linear_dgrad_bf16(logits, w["w_head"])
                K.rmsnorm_bwd(dxn, yc, w["final_norm"], rstd, dw=dw["final_norm"], accumulate=acc, out=dy[lo:hi])
                first = False
            loss.copy_(loss_dev, non_blocking=True)

    return RLHeadLoss


class RLTrainer:
    def __init__(self, family: str, cfg, *, device=None, budget_gib=None, objective: str = "ppo", lr: float = 2e-3, seed: int = 0):
        from dataflow_b200.blocks.base_blocks import HeadLoss
        from dataflow_b200.lowering.planning import plan_program
        from dataflow_b200.models.families import resolve_family
        from dataflow_b200.run.driver import Trainer
        self.fam = resolve_family(family)
        self.cfg = cfg
        bare = build_rl_program(self.fam, cfg)
        planned = plan_program(bare, None if budget_gib is None else int(budget_gib * (1 << 30)), leeway_bytes=0)
        self.tr = Trainer(family, cfg, budget_gib=budget_gib, device=device, hyper={"lr": lr, "weight_decay": 0.0}, seed=seed, planned=planned)
        head = make_rl_head(HeadLoss)(self.tr.dims, self.tr.layouts, self.tr.K, device, self.tr.hyper)
        head.objective = objective
        self.tr.resolver.table["rl_head_loss"] = head
        self.twin = self.fam.twin(cfg)

    def rollout(self, tokens, bounds, generator):
        """Sample one action per position from the current policy; returns (actions, log-probabilities)."""
        import torch
        self.tr.sync_to_host()
        self.twin.load_state_dict(self.fam.bridge(self.cfg, self.tr.views_of))
        with torch.no_grad():
            logits = self.twin(torch.as_tensor(tokens).long(), bounds)
            logp = torch.log_softmax(logits.float(), -1)
            actions = torch.multinomial(logp.exp(), 1, generator=generator)[:, 0]
        return actions.to(torch.int32), logp.gather(1, actions[:, None])[:, 0]

    def step(self, rounds):
        """``rounds``: list of (tokens, actions, advantages, old_logprobs) per round."""
        import torch
        tr = self.tr
        for r, (tk, act, adv, old) in enumerate(rounds):
            tr.put_round(r, tk, act)
            tr.host_tensor(f"advantages_0_{r}", (tr.T,), "fp32").copy_(torch.as_tensor(adv, dtype=torch.float32))
            tr.host_tensor(f"old_logprobs_0_{r}", (tr.T,), "fp32").copy_(torch.as_tensor(old, dtype=torch.float32))
        return tr.step(None)

    def close(self):
        self.tr.close()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--family", default="llama3")
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--objective", default="ppo", choices=["ppo", "reinforce"])
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args(argv)
    import torch
    from dataflow_b200.models.families import resolve_family
    cfg = dataclasses.replace(resolve_family(a.family).presets["tiny"](), dtype_policy="fp32" if a.device == "cpu" else "bf16_master")
    rl = RLTrainer(a.family, cfg, device=None if a.device == "cpu" else int(a.device), objective=a.objective, lr=5e-3)
    gen = torch.Generator().manual_seed(0)
    small = 16
    tr = rl.tr
    bounds = list(range(0, tr.T + 1, cfg.seq_len))
    for s in range(a.steps):
        rounds, rewards = [], []
        for r in range(tr.rounds):
            tk = torch.randint(0, small, (tr.T,), generator=gen, dtype=torch.int32)
            act, lp = rl.rollout(tk, bounds, gen)
            reward = (act == (tk + 1) % small).float()
            rewards.append(float(reward.mean()))
            rounds.append((tk, act, reward - reward.mean(), lp))
        loss = rl.step(rounds)
        print(f"step {s}: mean reward {sum(rewards) / len(rewards):.4f}  surrogate loss {loss:+.5f}")
    rl.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
