"""Model-family registry.  A family is a record of callables: config type, dims
derivation, lowering, seeded initial values, resolver construction, layouts.
Plugins register through ``register_family`` or the ``DATAFLOW_PLUGINS``
environment variable (comma-separated module names).  Contract parity: reference
``src/dataflow_training/model_families/families.py:68-536``.
"""
from __future__ import annotations

import importlib
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Mapping

from ..core import ObjectSpec, Program, TaskSpec


@dataclass(frozen=True)
class ModelFamily:
    name: str
    config_type: type
    derive_dims: Callable[[Any], Any]
    lower: Callable[..., Program]                       # lower(cfg, recompute_levels=None, hw=None) -> Program
    initial_values: Callable[..., None]                 # initial_values(program, cfg, views_of, seed)
    build_resolver: Callable[..., Callable]             # build_resolver(dims, hyper, kernels, device) -> resolver(task)
    family_layouts: Callable[[Any], Any]                # dims -> FamilyLayouts
    presets: Mapping[str, Callable[[], Any]] = field(default_factory=dict)
    twin: Callable[[Any], Any] | None = None            # cfg -> torch.nn.Module (pure-torch oracle)
    bridge: Callable[..., Mapping[str, Any]] | None = None   # engine views -> twin state_dict
    block_kinds: tuple[str, ...] = ()
    flops_per_token: Callable[[Any], float] | None = None


_FAMILIES: dict[str, ModelFamily] = {}
_BUILTIN = ("llama3", "gpt2", "qwen3", "olmoe", "qwen3moe", "dsv3", "dsv32", "glm52", "qwen35", "qwen35moe", "tp_mlp")


def register_family(fam: ModelFamily) -> ModelFamily:
    _FAMILIES[fam.name] = fam
    return fam


def load_plugins() -> list[str]:
    loaded = []
    for mod in filter(None, os.environ.get("DATAFLOW_PLUGINS", "").split(",")):
        importlib.import_module(mod.strip())
        loaded.append(mod.strip())
    try:
        from importlib.metadata import entry_points
        for ep in entry_points(group="dataflow.families"):
            ep.load()
            loaded.append(ep.name)
    except Exception:
        pass
    return loaded


def _ensure_builtin(name: str | None = None) -> None:
    for b in _BUILTIN:
        if (name is None or name == b) and b not in _FAMILIES:
            try:
                importlib.import_module(f"{__package__}.{b}")
            except ModuleNotFoundError as e:
                if f".{b}" not in str(e) and b not in str(e):
                    raise


def resolve_family(name: str) -> ModelFamily:
    if name not in _FAMILIES:
        _ensure_builtin(name)
    if name not in _FAMILIES:
        load_plugins()
    if name not in _FAMILIES:
        raise KeyError(f"unknown model family {name!r}; known: {sorted(_FAMILIES)}")
    return _FAMILIES[name]


def all_families() -> dict[str, ModelFamily]:
    _ensure_builtin()
    return dict(_FAMILIES)


def validate_family(name: str) -> list[str]:
    """Structural check without GPU math: lowers the ``tiny`` preset, validates the program,
    checks every compute key resolves and that layouts agree with object sizes."""
    from ..core import collect_problems
    fam = resolve_family(name)
    problems: list[str] = []
    if "tiny" not in fam.presets:
        return [f"family {name!r} has no 'tiny' preset"]
    cfg = fam.presets["tiny"]()
    prog = fam.lower(cfg)
    problems += collect_problems(prog)
    keys = {t.compute_block_key for t in prog.tasks}
    resolver = fam.build_resolver(fam.derive_dims(cfg), {}, None, None)
    for t in prog.tasks:
        try:
            resolver(t)
        except Exception as e:      # noqa: BLE001
            problems.append(f"task {t.id}: key {t.compute_block_key!r} does not resolve: {e}")
            break
    lay = fam.family_layouts(fam.derive_dims(cfg))
    sizes = prog.object_sizes()
    for oid, layout in lay.object_layouts(prog).items():
        if oid in sizes and layout.size_bytes != sizes[oid]:
            problems.append(f"object {oid}: layout {layout.size_bytes} B != program {sizes[oid]} B")
    if not keys:
        problems.append("program has no tasks")
    return problems


def build_init_program(program: Program, name: str | None = None) -> Program:
    """One HOST task ``family_init_0`` whose inputs/mutations are the training program's
    persistent initial objects (init-as-program)."""
    objs = tuple(o for o in program.initial_objects if o.persistent)
    seen, uniq = set(), []
    for o in objs:
        if o.id not in seen:
            seen.add(o.id)
            uniq.append(ObjectSpec(o.id, o.size_bytes, "backing", o.role, o.tensor, True))
    ids = tuple(o.id for o in uniq)
    task = TaskSpec("family_init_0", inputs=ids, mutates=ids, compute_block_key="family_init", host=True,
                    group="init")
    return Program(name or f"{program.name}:init", tuple(uniq), (task,), {i: "backing" for i in ids})
