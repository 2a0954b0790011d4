"""Frozen training: which parts of a model take no update, and the program that results.

``derive_freeze_plan`` reads an optimizer policy (``blocks.optim.freeze(...)`` composes them) against a family's
field lists and says, per layer, which fields are frozen and whether the whole layer is.  ``to_frozen_form`` rewrites
a lowered (bare, single-rank) program accordingly:

* a fully frozen layer loses its optimizer task, its gradient object ``dW_i`` and its optimizer state ``O_i``; its
  backward still runs (the layers below need the input gradient) at the data-gradient share of its cost;
* a frozen PREFIX (embedding frozen and layers ``0 .. k-1`` frozen) loses backward and recompute tasks altogether, and
  the saved contexts of those layers are never produced;
* partially frozen layers keep their tasks; their ``block_params["frozen_fields"]`` tells the executables which
  fields to skip (the optimizer leaves them untouched and wgrad for them is not computed).

Reference role: ``src/dataflow_training/lowering/freeze_plan.py:71,140`` (``FreezePlan``, ``derive_freeze_plan``) and
``freeze_program.py:40`` (``to_frozen_form``).
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field, replace
from typing import Mapping, Sequence

from ..blocks.optim import OptPolicy, resolve_opt_policy

DGRAD_SHARE = 0.55          # backward cost of a layer whose weight gradients are all skipped


@dataclass(frozen=True)
class FreezePlan:
    n_layers: int
    frozen_fields: Mapping[int, tuple[str, ...]] = field(default_factory=dict)     # layer -> frozen field names
    frozen_layers: tuple[int, ...] = ()                                             # every field frozen
    embed_frozen: bool = False
    head_frozen: bool = False

    @property
    def frozen_prefix(self) -> int:
        """Number of leading layers that need no backward at all."""
        if not self.embed_frozen:
            return 0
        k = 0
        while k < self.n_layers and k in self.frozen_layers:
            k += 1
        return k

    @property
    def trainable_layers(self) -> tuple[int, ...]:
        return tuple(i for i in range(self.n_layers) if i not in self.frozen_layers)

    def describe(self) -> str:
        return (f"{len(self.frozen_layers)}/{self.n_layers} layers frozen, prefix {self.frozen_prefix}, "
                f"embed {'frozen' if self.embed_frozen else 'trained'}, head {'frozen' if self.head_frozen else 'trained'}")


def derive_freeze_plan(policy, n_layers: int, block_fields: Sequence, embed_fields: Sequence = (), head_fields: Sequence = ()) -> FreezePlan:
    """``*_fields``: objects with ``.name`` and ``.kind`` (the family's field lists)."""
    pol: OptPolicy = resolve_opt_policy(policy)
    per_layer, whole = {}, []
    for i in range(n_layers):
        fr = tuple(f.name for f in block_fields if pol.rule_for(f.name, i, getattr(f, "kind", "matrix")) == "frozen")
        if fr:
            per_layer[i] = fr
        if block_fields and len(fr) == len(block_fields):
            whole.append(i)

    def all_frozen(fields, layer):
        return bool(fields) and all(pol.rule_for(f.name, layer, getattr(f, "kind", "matrix")) == "frozen" for f in fields)

    return FreezePlan(n_layers, per_layer, tuple(whole), all_frozen(embed_fields, "embed"), all_frozen(head_fields, "head"))


def _layer_of(task) -> int | None:
    v = task.block_params.get("layer") if task.block_params else None
    return int(v) if v is not None else None


def to_frozen_form(program, plan: FreezePlan):
    """Returns the rewritten program (bare).  Refuses sharded (ZeRO) programs: freeze first, shard after."""
    if (program.metadata or {}).get("zero"):
        raise ValueError("to_frozen_form works on the single-rank lowering; apply it before sharding")
    if program.is_annotated():
        raise ValueError("to_frozen_form needs the bare program: plan after freezing")
    prefix = plan.frozen_prefix
    dead: set[str] = set()
    for oid in program.object_sizes():
        m = _GRAD.match(oid)
        if m and int(m.group(1)) in plan.frozen_layers:
            dead.add(oid)
        if plan.embed_frozen and oid.startswith("dW_embed"):
            dead.add(oid)
        if plan.head_frozen and oid.startswith("dW_head"):
            dead.add(oid)
    dead.update(f"O_{i}" for i in plan.frozen_layers)
    if plan.embed_frozen:
        dead.add("O_embed")
    if plan.head_frozen:
        dead.add("O_head")
    tasks = []
    for t in program.tasks:
        key, layer = t.compute_block_key or "", _layer_of(t)
        if key.startswith("optimizer"):
            target = t.block_params.get("target")
            if (layer is not None and layer in plan.frozen_layers) or (target == "embed" and plan.embed_frozen) or \
                    (target == "head" and plan.head_frozen):
                continue
        if layer is not None and layer < prefix and (key.endswith("_bwd") or key.endswith("_recompute")):
            continue
        if key == "embed_bwd" and plan.embed_frozen:
            continue
        tasks.append(t)
    # objects only the dropped tasks produced or consumed disappear with them
    consumed = {i for t in tasks for i in t.inputs}
    out_tasks = []
    for t in tasks:
        key, layer = t.compute_block_key or "", _layer_of(t)
        outs = tuple(o for o in t.outputs if o.id not in dead and (o.id in consumed or o.id in program.final_locations
                                                                   or not _is_transient(o.id)))
        ins = tuple(i for i in t.inputs if i not in dead)
        mut = tuple(m for m in t.mutates if m not in dead)
        params = dict(t.block_params)
        runtime = t.runtime_us
        if layer is not None and layer in plan.frozen_fields and (key.endswith("_bwd") or key.startswith("optimizer")):
            params["frozen_fields"] = list(plan.frozen_fields[layer])
        if layer is not None and layer in plan.frozen_layers and key.endswith("_bwd"):
            runtime = t.runtime_us * DGRAD_SHARE
        out_tasks.append(replace(t, inputs=ins, outputs=outs, mutates=mut, block_params=params, runtime_us=runtime))
    initial = tuple(o for o in program.initial_objects if o.id not in dead)
    final = {k: v for k, v in program.final_locations.items() if k not in dead}
    rewrites = tuple(r for r in program.recompute_rewrites
                     if not any(r.f_task_id == t.id and (_layer_of(t) or 0) < prefix for t in program.tasks))
    md = dict(program.metadata or {})
    md["freeze"] = {"frozen_layers": list(plan.frozen_layers), "prefix": prefix, "embed": plan.embed_frozen, "head": plan.head_frozen}
    return replace(program, initial_objects=initial, tasks=tuple(out_tasks), final_locations=final, recompute_rewrites=rewrites,
                   metadata=md)


_GRAD = re.compile(r"^dW_\d+_(\d+)$")


def _is_transient(oid: str) -> bool:
    """Saved contexts and input gradients: produced only for a later task of the same step."""
    return oid.startswith(("A_", "Ap_", "AuxTemp", "dy_"))
