"""Canonical JSON form of a Program (wire-compatible with ``dataflow-rt/v1``).

Encoding is table-driven: each dataclass lists ``(field, default, codec)``; a
field equal to its default is left out, so a bare program and its content
hash never change because an optional field exists.  ``persistent`` and
``host`` appear only when true.  Same key names and omission rules as the
reference's ``src/dataflow/core/jsonio.py:110-238``.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any, Callable

from .program import (SCHEMA_VERSION, ObjectSpec, OutputSpec, Program, RecomputeOption,
                      RecomputeRewrite, TaskSpec, TransferDirective)
from .types import TensorMeta

_ALWAYS = object()          # sentinel: emit regardless of value


def _enc_tensor(t: TensorMeta | None):
    if t is None:
        return None
    d: dict[str, Any] = {}
    if t.dtype is not None:
        d["dtype"] = t.dtype
    if t.shape is not None:
        d["shape"] = list(t.shape)
    if t.strides is not None:
        d["strides"] = list(t.strides)
    return d or None


def _dec_tensor(d):
    if not d:
        return None
    return TensorMeta(dtype=d.get("dtype"),
                      shape=tuple(d["shape"]) if d.get("shape") is not None else None,
                      strides=tuple(d["strides"]) if d.get("strides") is not None else None)


def _enc_object(o) -> dict[str, Any]:
    d = {"id": o.id, "size_bytes": int(o.size_bytes), "location": o.location, "role": o.role}
    if getattr(o, "persistent", False):
        d["persistent"] = True
    t = _enc_tensor(o.tensor)
    if t is not None:
        d["tensor"] = t
    return d


def _dec_initial(d) -> ObjectSpec:
    return ObjectSpec(id=d["id"], size_bytes=int(d["size_bytes"]),
                      location=d.get("location", "backing"), role=d.get("role", "other"),
                      tensor=_dec_tensor(d.get("tensor")), persistent=bool(d.get("persistent", False)))


def _dec_output(d) -> OutputSpec:
    return OutputSpec(id=d["id"], size_bytes=int(d["size_bytes"]),
                      location=d.get("location", "fast"), role=d.get("role", "other"),
                      tensor=_dec_tensor(d.get("tensor")))


def _enc_directive(t: TransferDirective):
    d: dict[str, Any] = {"object_id": t.object_id}
    if t.runtime_us is not None:
        d["runtime_us"] = t.runtime_us
    return d


def _dec_directive(d) -> TransferDirective:
    if isinstance(d, str):
        return TransferDirective(d)
    return TransferDirective(object_id=d["object_id"], runtime_us=d.get("runtime_us"))


# (field, skip-if-equal-to, encoder, decoder)
_TASK_FIELDS: tuple[tuple[str, Any, Callable, Callable], ...] = (
    ("id", _ALWAYS, str, str),
    ("runtime_us", _ALWAYS, lambda v: v, float),
    ("workspace_bytes", 0, int, int),
    ("inputs", (), list, tuple),
    ("outputs", (), lambda v: [_enc_object(o) for o in v], lambda v: tuple(_dec_output(o) for o in v)),
    ("mutates", (), list, tuple),
    ("group", "compute", str, str),
    ("compute_block_key", None, lambda v: v, lambda v: v),
    ("block_params", {}, dict, dict),
    ("comm_groups", {}, dict, dict),
    ("releases_after", (), list, tuple),
    ("offload_after", (), lambda v: [_enc_directive(x) for x in v], lambda v: tuple(_dec_directive(x) for x in v)),
    ("prefetch_after", (), lambda v: [_enc_directive(x) for x in v], lambda v: tuple(_dec_directive(x) for x in v)),
    ("label", None, lambda v: v, lambda v: v),
    ("metadata", {}, dict, dict),
    ("host", False, bool, bool),
)


def _enc_task(t: TaskSpec) -> dict[str, Any]:
    d: dict[str, Any] = {}
    for name, skip, enc, _ in _TASK_FIELDS:
        v = getattr(t, name)
        if skip is not _ALWAYS:
            if v is None and skip is None:
                continue
            if skip is not None and (v == skip or (not v and not skip)):
                continue
        d[name] = enc(v)
    return d


def _dec_task(d) -> TaskSpec:
    kw: dict[str, Any] = {}
    for name, _skip, _enc, dec in _TASK_FIELDS:
        if name in d and d[name] is not None:
            kw[name] = dec(d[name])
    return TaskSpec(**kw)


def _enc_rewrite(rw: RecomputeRewrite):
    return {
        "object_id": rw.object_id, "f_task_id": rw.f_task_id, "r_task_id": rw.r_task_id,
        "options": [{"level": o.level, "saved_bytes": o.saved_bytes,
                     "recompute_us": o.recompute_us, "label": o.label} for o in rw.options],
        "f_compute_block_key": rw.f_compute_block_key,
        "r_compute_block_key": rw.r_compute_block_key,
        "group_key": rw.group_key,
    }


def _dec_rewrite(d) -> RecomputeRewrite:
    return RecomputeRewrite(
        object_id=d["object_id"], f_task_id=d["f_task_id"], r_task_id=d["r_task_id"],
        options=tuple(RecomputeOption(int(o["level"]), int(o["saved_bytes"]),
                                      float(o["recompute_us"]), o.get("label", ""))
                      for o in d["options"]),
        f_compute_block_key=d.get("f_compute_block_key", ""),
        r_compute_block_key=d.get("r_compute_block_key", ""),
        group_key=d.get("group_key", ""))


_OPTIONAL_TOP = ("fast_memory_capacity", "backing_memory_capacity",
                 "bandwidth_from_slow", "bandwidth_to_slow")


def program_to_dict(p: Program) -> dict[str, Any]:
    d: dict[str, Any] = {
        "schema_version": p.schema_version,
        "name": p.name,
        "initial_objects": [_enc_object(o) for o in p.initial_objects],
        "tasks": [_enc_task(t) for t in p.tasks],
    }
    if p.final_locations:
        d["final_locations"] = dict(p.final_locations)
    for k in _OPTIONAL_TOP:
        v = getattr(p, k)
        if v is not None:
            d[k] = v
    if p.recompute_rewrites:
        d["recompute_rewrites"] = [_enc_rewrite(r) for r in p.recompute_rewrites]
    if p.metadata:
        d["metadata"] = dict(p.metadata)
    return d


def program_from_dict(d: dict[str, Any]) -> Program:
    """A ``Program`` from its JSON form.  A document that is not one (a key missing, a list where an object belongs, a string
    where a number belongs) is refused with a ``ValueError`` that says where, never with the ``KeyError`` / ``TypeError``
    the decoding happened to trip over."""
    if not isinstance(d, dict):
        raise ValueError(f"not a {SCHEMA_VERSION} program: the document is a {type(d).__name__}, not an object")
    try:
        return _program_from_dict(d)
    except (KeyError, TypeError, AttributeError, IndexError) as e:
        what = f"key {e.args[0]!r} is missing" if isinstance(e, KeyError) and e.args else f"{type(e).__name__}: {e}"
        raise ValueError(f"not a {SCHEMA_VERSION} program: {what}") from None


def _program_from_dict(d: dict[str, Any]) -> Program:
    version = d.get("schema_version", SCHEMA_VERSION)
    if version != SCHEMA_VERSION:
        raise ValueError(f"unsupported schema_version {version!r}; expected {SCHEMA_VERSION!r}")
    return Program(
        name=d["name"],
        initial_objects=tuple(_dec_initial(o) for o in d.get("initial_objects", ())),
        tasks=tuple(_dec_task(t) for t in d.get("tasks", ())),
        final_locations=dict(d.get("final_locations", {})),
        **{k: d.get(k) for k in _OPTIONAL_TOP},
        recompute_rewrites=tuple(_dec_rewrite(r) for r in d.get("recompute_rewrites", ())),
        metadata=dict(d.get("metadata", {})),
        schema_version=version,
    )


def canonical_json(obj: Any) -> str:
    """Key-sorted, separator-tight JSON: the byte string content ids hash."""
    return json.dumps(obj, sort_keys=True, separators=(",", ":"))


def program_content_id(program_or_dict) -> str:
    """``"p-" + sha256(canonical JSON)[:12]`` — reference ``service/wire.py:37-48``."""
    d = program_or_dict if isinstance(program_or_dict, dict) else program_to_dict(program_or_dict)
    return "p-" + hashlib.sha256(canonical_json(d).encode()).hexdigest()[:12]


def save_program(program: Program, path) -> None:
    Path(path).write_text(json.dumps(program_to_dict(program), indent=2) + "\n")


def load_program(path) -> Program:
    return program_from_dict(json.loads(Path(path).read_text()))
