"""Preset resolution and config (de)serialisation.  ``resolve_preset("llama3_8b")`` or
``"family:preset"``; ``cfg_dict`` / ``cfg_from_dict`` carry a config over the wire so the daemon
rebuilds identical dims.  Parity: reference ``src/dataflow_training/run/presets.py:96-216``."""
from __future__ import annotations

import dataclasses
from typing import Any

from ..blocks.layouts import DTypePolicy
from ..models.families import all_families, resolve_family


def resolve_preset(name: str):
    """Returns ``(family_name, config)``."""
    if ":" in name:
        fam, preset = name.split(":", 1)
        return fam, resolve_family(fam).presets[preset]()
    hits = [(f.name, f.presets[name]) for f in all_families().values() if name in f.presets]
    if not hits:
        raise KeyError(f"unknown preset {name!r}")
    if len(hits) > 1:
        raise KeyError(f"preset {name!r} exists in several families {[h[0] for h in hits]}: qualify it as 'family:{name}'")
    return hits[0][0], hits[0][1]()


def cfg_dict(cfg) -> dict[str, Any]:
    d = {}
    for f in dataclasses.fields(cfg):
        v = getattr(cfg, f.name)
        d[f.name] = v.to_dict() if isinstance(v, DTypePolicy) else v
    return d


def cfg_from_dict(fam, d: dict[str, Any]):
    names = {f.name for f in dataclasses.fields(fam.config_type)}
    return fam.config_type(**{k: v for k, v in d.items() if k in names})
