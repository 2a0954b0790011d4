"""The checkpoint record: ``checkpoint_record.json``, the one cross-source file of a checkpoint.

Everything else in a step directory is engine snapshots and program dumps.  The record is written atomically
and LAST — its presence is the completeness marker.  ``validate_record`` enforces: full coverage of every
logical object's byte span (a gap is refused by name and range); overlap only as exact-span replicas with
equal hashes (the drift certificate), partial overlaps refused; with field schemas, slice endpoints on element
boundaries.  ``scheme``, ``client_payload``, ``summary`` and ``launch`` are opaque.
Contract parity: reference ``src/dataflow/checkpoint/record.py:22-120`` and ``docs/checkpointing.md:226-304``.
"""
from __future__ import annotations

import json
import os
from typing import Any, Mapping

RECORD_SCHEMA = "dataflow-checkpoint/v1"
RECORD_FILE = "checkpoint_record.json"


class RecordError(ValueError):
    pass


def build_record(*, step: int, seed: int, scheme: Mapping[str, Any], logical_objects: Mapping[str, Mapping[str, Any]],
                 snapshots: list[Mapping[str, Any]], slices: Mapping[str, list[Mapping[str, Any]]],
                 engine_spec: Mapping[str, Any] | None = None, client_payload: Any = None, summary: Any = None,
                 launch: Any = None) -> dict:
    rec = {"schema": RECORD_SCHEMA, "step": int(step), "seed": int(seed), "scheme": dict(scheme),
           "logical_objects": {k: dict(v) for k, v in logical_objects.items()},
           "snapshots": [dict(s) for s in snapshots],
           "slices": {k: [dict(x) for x in v] for k, v in slices.items()},
           "engine_spec": dict(engine_spec or {}), "client_payload": client_payload, "summary": summary, "launch": launch}
    validate_record(rec)
    return rec


def validate_record(rec: Mapping[str, Any], field_schemas: Mapping[str, Mapping[str, Any]] | None = None) -> None:
    if rec.get("schema") != RECORD_SCHEMA:
        raise RecordError(f"foreign checkpoint schema {rec.get('schema')!r} (this layer reads {RECORD_SCHEMA!r} only)")
    snaps = rec.get("snapshots") or []
    objs = rec.get("logical_objects") or {}
    slices = rec.get("slices") or {}
    for i, s in enumerate(snaps):
        if "path" not in s or "objects" not in s:
            raise RecordError(f"snapshot {i} lacks path / resident-object inventory")
    for oid in slices:
        if oid not in objs:
            raise RecordError(f"slices name {oid!r}, which is not a logical object of the record")
    for oid, meta in objs.items():
        total = int(meta["bytes"])
        ents = slices.get(oid) or []
        if not ents and total:
            raise RecordError(f"{oid}: no slices cover its {total} bytes")
        spans: dict[tuple[int, int], list[Mapping[str, Any]]] = {}
        for e in ents:
            si = int(e["snapshot"])
            if not 0 <= si < len(snaps):
                raise RecordError(f"{oid}: slice names snapshot {si}, the record has {len(snaps)}")
            a, b = (int(x) for x in e["object_range"])
            sa, sb = (int(x) for x in e["snapshot_range"])
            if not (0 <= a < b <= total) or sb - sa != b - a or sa < 0:
                raise RecordError(f"{oid}: bad ranges object {[a, b]} snapshot {[sa, sb]} for a {total}-byte object")
            base = oid.split("@", 1)[0]
            holder = snaps[si]["objects"]
            local = e.get("snapshot_object")
            held = holder.get(local) if local else holder.get(oid, holder.get(base))
            if held is None or sb > int(held):
                raise RecordError(f"{oid}: snapshot {si} ({snaps[si]['path']}) does not hold bytes {[sa, sb]} of it")
            spans.setdefault((a, b), []).append(e)
        keys = sorted(spans)
        pos = 0
        for a, b in keys:
            if a < pos:
                raise RecordError(f"{oid}: slices {[a, b]} partially overlap earlier bytes (replicas must span identically)")
            if a > pos:
                raise RecordError(f"{oid}: bytes [{pos}, {a}) are covered by no slice")
            pos = b
        if pos != total:
            raise RecordError(f"{oid}: bytes [{pos}, {total}) are covered by no slice")
        for (a, b), group in spans.items():
            hashes = {e.get("hash") for e in group}
            if len(group) > 1 and (len(hashes) != 1 or None in hashes):
                raise RecordError(f"{oid}: replicas of bytes {[a, b]} differ (hashes {sorted(map(str, hashes))}): state drifted")
        schema = (field_schemas or {}).get(oid)
        if schema:
            if meta.get("schema_digest") not in (None, schema.get("digest")):
                raise RecordError(f"{oid}: field-schema digest {meta.get('schema_digest')} != {schema.get('digest')}")
            item = int(schema.get("element_bytes", 1))
            for a, b in keys:
                if a % item or b % item:
                    raise RecordError(f"{oid}: slice {[a, b]} does not land on {item}-byte element boundaries")


def write_record(step_dir: str, rec: Mapping[str, Any]) -> str:
    validate_record(rec)
    path = os.path.join(step_dir, RECORD_FILE)
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        json.dump(rec, f, indent=1, sort_keys=True)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)
    return path


def read_record(step_dir: str, field_schemas: Mapping[str, Mapping[str, Any]] | None = None) -> dict:
    path = os.path.join(step_dir, RECORD_FILE)
    if not os.path.exists(path):
        raise RecordError(f"{step_dir}: no {RECORD_FILE} — not a complete checkpoint")
    try:
        with open(path) as f:
            rec = json.load(f)
    except (ValueError, OSError) as e:
        raise RecordError(f"{path} is damaged ({type(e).__name__}: {e}) — not a complete checkpoint") from None
    validate_record(rec, field_schemas)
    return rec


def has_record(step_dir: str) -> bool:
    """True when the directory holds a record that parses.  The record is written last, so its presence means every slice
    was written; a record that does not parse (a damaged disk, a copy cut short) makes the directory no checkpoint at all,
    and resuming from "latest" then goes to the step before."""
    path = os.path.join(step_dir, RECORD_FILE)
    if not os.path.exists(path):
        return False
    try:
        with open(path) as f:
            return isinstance(json.load(f), dict)
    except (ValueError, OSError):
        return False
