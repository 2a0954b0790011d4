"""Program surgery for policy-gradient training on any registered family.

The supervised lowering of a family is turned into an RL step by three edits:

* every block forward keeps NOTHING (recompute level 2 everywhere): a rollout batch is long and only sampled once, so
  the saved contexts of the supervised step are replaced by a recompute task in front of every backward;
* the cross-entropy head is replaced by ``rl_head_loss`` — same GEMMs and norm backward, policy-gradient loss in the
  middle (``rl_ops.policy_loss_fwd_bwd``);
* every round gets two more inputs, ``advantages_{s}_{r}`` and ``old_logprobs_{s}_{r}`` (fp32 per token), which the
  head reads; ``targets_{s}_{r}`` carries the sampled actions (-1 where a token is not a decision).

Reference role: ``examples/rl_training/builder.py:34``.
"""
from __future__ import annotations

import dataclasses


def build_rl_program(family, cfg, hw=None, **lower_kwargs):
    """Returns the bare RL program of ``cfg`` (plan it with ``lowering.planning.plan_program``)."""
    from dataflow_b200.core.program import ObjectSpec
    from dataflow_b200.models.families import resolve_family
    fam = resolve_family(family) if isinstance(family, str) else family
    levels = {i: 2 for i in range(cfg.n_layers)}
    prog = fam.lower(cfg, recompute_levels=levels, hw=hw, **lower_kwargs)
    tokens = prog.metadata["tokens_per_round"]
    extra, tasks = [], []
    for t in prog.tasks:
        if t.compute_block_key == "head_loss":
            s, r = t.id.split("_")[-2:]
            adv, old = f"advantages_{s}_{r}", f"old_logprobs_{s}_{r}"
            extra += [ObjectSpec(adv, tokens * 4, "backing", "input"), ObjectSpec(old, tokens * 4, "backing", "input")]
            t = dataclasses.replace(t, compute_block_key="rl_head_loss", inputs=tuple(t.inputs) + (adv, old))
        tasks.append(t)
    md = dict(prog.metadata, objective="policy_gradient")
    return dataclasses.replace(prog, initial_objects=tuple(prog.initial_objects) + tuple(extra), tasks=tuple(tasks), metadata=md)
