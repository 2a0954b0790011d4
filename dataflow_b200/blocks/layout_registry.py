"""The named layout registry: every family's packed weight layouts as keyed, validated, addressable artifacts — the
coordinate system sharding plans, responsibility maps and checkpoints speak.

Keys are ``"<family>/<kind>"`` for the kinds of layers a configuration has (one entry per DISTINCT layout; ``roots``
lists the layers it backs) plus ``"<family>/embed"`` and ``"<family>/head"``.  An entry is the layout's field table as
data: name, shape, dtype, byte offset, byte size, role, init tag.  The registry is derived from the family's own layouts —
there is no second source of truth — and ``validate`` makes "well formed" checkable: unique field names, monotone
non-overlapping offsets, positive sizes, fields inside the object.  ``layouts_digest`` pins the whole surface (initial
bytes ride field order, sharding rides offsets): the digest gate in the tests is what lets layout code change form
without changing what it produces.
Role parity: reference ``src/dataflow_training/model_families/layout_registry.py:1-133``.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass
from typing import Any


@dataclass(frozen=True)
class RegisteredLayout:
    key: str                      # "<family>/<kind>"
    family: str
    kind: str
    fields: tuple                 # ((name, shape, dtype, offset_bytes, size_bytes, role, init), ...)
    total_bytes: int
    roots: tuple                  # object ids this layout backs ("W_0", "W_3", ... or "W_embed")

    def field(self, name: str) -> tuple:
        for f in self.fields:
            if f[0] == name:
                return f
        raise KeyError(f"{self.key} has no field {name!r}")

    def to_dict(self) -> dict:
        return {"key": self.key, "total_bytes": self.total_bytes, "roots": list(self.roots),
                "fields": [[n, list(sh), dt, off, sz, role, init] for n, sh, dt, off, sz, role, init in self.fields]}


def field_table(layout) -> tuple:
    offs = layout.offsets()
    return tuple((f.name, tuple(int(x) for x in f.shape), f.dtype, int(offs[f.name]), int(f.nbytes), f.kind, f.init) for f in layout.fields)


def registered_layouts(family, cfg) -> dict[str, RegisteredLayout]:
    """``{key: RegisteredLayout}`` of ``cfg``'s weight objects (layer kinds, embed, head)."""
    from ..models.families import resolve_family
    fam = resolve_family(family) if isinstance(family, str) else family
    dims = fam.derive_dims(cfg)
    lay = fam.family_layouts(dims)
    prog = fam.lower(cfg)
    kinds = list(getattr(dims, "kinds", ()) or ())
    out: dict[str, RegisteredLayout] = {}
    by_table: dict[tuple, str] = {}
    for o in prog.initial_objects:
        if not (o.persistent and o.id.startswith("W_")):
            continue
        tail = o.id[2:]
        layout = lay.layout_of(o.id)
        table = field_table(layout)
        if tail.isdigit():
            kind = kinds[int(tail)] if kinds else "block"
        else:
            kind = tail
        key = f"{fam.name}/{kind}"
        seen = by_table.get((key, table))
        if seen is None and key in out:                       # the same kind name with another table (e.g. the last layer differs)
            n = 2
            while f"{key}#{n}" in out:
                n += 1
            key = f"{key}#{n}"
        if (key, table) in by_table or seen is not None:
            k = seen or key
            e = out[k]
            out[k] = RegisteredLayout(e.key, e.family, e.kind, e.fields, e.total_bytes, e.roots + (o.id,))
            continue
        by_table[(key, table)] = key
        out[key] = RegisteredLayout(key, fam.name, kind, table, int(layout.size_bytes), (o.id,))
    return out


def validate(entry: RegisteredLayout) -> list[str]:
    problems = []
    names = [f[0] for f in entry.fields]
    if len(set(names)) != len(names):
        problems.append(f"{entry.key}: duplicate field names")
    end = 0
    for name, shape, dtype, off, size, role, init in entry.fields:
        if size <= 0:
            problems.append(f"{entry.key}.{name}: size {size}")
        if off < end:
            problems.append(f"{entry.key}.{name}: offset {off} overlaps the previous field (ends at {end})")
        if off % 256:
            problems.append(f"{entry.key}.{name}: offset {off} is not 256-byte aligned")
        end = off + size
    if end > entry.total_bytes:
        problems.append(f"{entry.key}: fields end at {end}, the object has {entry.total_bytes} bytes")
    return problems


def layouts_digest(family, cfg) -> str:
    reg = registered_layouts(family, cfg)
    blob = json.dumps({k: v.to_dict() for k, v in sorted(reg.items())}, sort_keys=True, separators=(",", ":"))
    return hashlib.sha256(blob.encode()).hexdigest()


def describe(family, cfg) -> dict[str, Any]:
    """The registry as plain data (tools, docs)."""
    return {k: v.to_dict() for k, v in sorted(registered_layouts(family, cfg).items())}
