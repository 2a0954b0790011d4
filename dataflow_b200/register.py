"""Registers the workload with the service: resolver kind ``"model_family"`` (spec =
``{"kind", "family", "cfg", "hyper"}``) and the HOST init task (``family_init``) that fills a
training program's persistent objects with the family's seeded initial values directly in the
store's extents (init-as-program).  Role parity: reference ``src/dataflow_training/register.py:40-122``."""
from __future__ import annotations

from typing import Any, Mapping


def canonical_spec(family: str, cfg, hyper: Mapping[str, Any] | None = None, seed: int | None = None) -> dict:
    from .run.presets import cfg_dict
    spec = {"kind": "model_family", "family": family, "cfg": cfg_dict(cfg), "hyper": dict(hyper or {})}
    if seed is not None:
        spec["seed"] = int(seed)
    return spec


class FamilyInitExecutable:
    def __init__(self, fam, cfg, seed: int, init_policy=None):
        self.fam, self.cfg, self.seed, self.init_policy = fam, cfg, seed, init_policy

    def launch(self, ctx) -> None:
        bufs = {b.object_id: b for b in ctx.inputs}
        program = self.fam.lower(self.cfg)

        def views_of(oid, layout):
            return layout.views(bufs[oid], None)
        import dataclasses
        keep = tuple(o for o in program.initial_objects if o.id in bufs)
        from .blocks.init_policy import init_scope
        with init_scope(self.init_policy):           # the resolver spec's hyper["init_policy"]: rules by field name and layer
            self.fam.initial_values(dataclasses.replace(program, initial_objects=keep), self.cfg, views_of, self.seed)


def build_model_family_resolver(spec: Mapping[str, Any], env):
    from .models.families import resolve_family
    from .ops import resolve_kernels
    from .run.presets import cfg_from_dict
    fam = resolve_family(spec["family"])
    cfg = cfg_from_dict(fam, spec["cfg"])
    device = getattr(env, "device", None)
    kernel_set = getattr(env, "kernel_set", None)
    K = resolve_kernels(kernel_set=("eager" if device is None and kernel_set is None else kernel_set))
    hyper = dict(spec.get("hyper") or {})
    hyper.setdefault("optimizer", getattr(cfg, "optimizer", "adamw"))
    if hasattr(cfg, "policy"):
        hyper.setdefault("dtype_policy", cfg.policy().to_dict())
    dims = fam.derive_dims(cfg)
    inner = fam.build_resolver(dims, hyper, K, device)
    dp = spec.get("dp")
    if dp and dp.get("mode", "co") in ("co", "dp"):
        # replicas over a peer group of the daemons (fleet mode): every optimizer task first sums its gradient object over
        # the group named here; the handle comes from the daemon's peer plane (``ctx.groups[name]``)
        from types import SimpleNamespace
        from .parallel.zero import replicate_gradients
        layouts = fam.family_layouts(dims, cfg.policy() if hasattr(cfg, "policy") else None, hyper["optimizer"])
        replicate_gradients(SimpleNamespace(resolver=inner, layouts=layouts), dp.get("group", "dp"))
    elif dp:
        raise ValueError(f"fleet mode runs replicas (dp mode 'co'); {dp.get('mode')!r} needs the in-process launcher")
    init = FamilyInitExecutable(fam, cfg, int(spec.get("seed", 0)), (spec.get("hyper") or {}).get("init_policy"))

    def resolver(task):
        if task.compute_block_key == "family_init":
            return init
        return inner(task)
    return resolver


def register_all() -> None:
    from .service.registry import register_program_resolver
    register_program_resolver("model_family", build_model_family_resolver)
