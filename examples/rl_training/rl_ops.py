"""Policy-gradient losses on the head's logits, written like the fused cross-entropy: one pass gives the loss and
replaces the logits by their gradient.

    REINFORCE      L = -A * log pi(a)
    PPO (clipped)  L = -min(r A, clip(r, 1 - eps, 1 + eps) A),   r = pi(a) / pi_old(a)

``actions < 0`` marks rows that carry no decision (prompt tokens, padding).  Reference role:
``examples/rl_training/rl_ops.py:33-106``.
"""
from __future__ import annotations

import torch


def policy_loss_fwd_bwd(logits, actions, advantages, old_logprobs, total_rows: float, loss_out, *, objective: str = "ppo",
                        clip_eps: float = 0.2, accumulate: bool = False):
    """In place: ``logits`` (rows, vocab) become d(loss)/d(logits); ``loss_out`` (1,) fp32 receives (or accumulates) the
    summed loss divided by ``total_rows``."""
    z = logits.float()
    valid = actions >= 0
    a = actions.clamp(min=0).long()
    logp_all = torch.log_softmax(z, dim=-1)
    lp = logp_all.gather(1, a[:, None])[:, 0]
    adv = advantages.float()
    if objective == "reinforce":
        loss = -adv * lp
        dlp = -adv
    elif objective == "ppo":
        ratio = torch.exp(lp - old_logprobs.float())
        clipped = ratio.clamp(1 - clip_eps, 1 + clip_eps)
        un, cl = ratio * adv, clipped * adv
        take_un = un <= cl                                     # min picks the unclipped branch: gradient flows through r
        loss = -torch.where(take_un, un, cl)
        inside = (ratio > 1 - clip_eps) & (ratio < 1 + clip_eps)
        dlp = -torch.where(take_un | inside, ratio * adv, torch.zeros_like(adv))
    else:
        raise KeyError(f"objective {objective!r} (ppo | reinforce)")
    scale = valid.float() / float(total_rows)
    total = (loss * scale).sum().reshape(1)
    if accumulate:
        loss_out.add_(total.to(loss_out.dtype))
    else:
        loss_out.copy_(total.to(loss_out.dtype))
    # d lp / d logits = onehot(a) - softmax
    grad = -torch.exp(logp_all)
    grad.scatter_add_(1, a[:, None], torch.ones_like(lp)[:, None])
    logits.copy_((grad * (dlp * scale)[:, None]).to(logits.dtype))
    return lp.detach()
