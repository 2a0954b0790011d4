"""From a record and a request to per-snapshot restore plans.

``targets`` may be ``"all"``, a list of logical ids, a ``{source: ids}`` dict (the rank view: every source gets
its own objects, bare ids resolving to source-qualified ones ``Aux_0@1`` where those exist) or a Program (its
persisted objects).  Reader rule for replicated spans: the lowest-index covering snapshot.
Contract parity: reference ``src/dataflow/checkpoint/targets.py:24-220``.
"""
from __future__ import annotations

from typing import Any, Iterable, Mapping


def persisted_objects(program) -> dict[str, int]:
    """Ids and sizes of a program's persistent initial objects."""
    return {o.id: int(o.size_bytes) for o in program.initial_objects if getattr(o, "persistent", False)}


def source_resident_bytes(record: Mapping[str, Any]) -> dict[str, int]:
    return {str(s.get("source", i)): int(sum(int(v) for v in s["objects"].values()))
            for i, s in enumerate(record["snapshots"])}


def _qualified(record, oid: str, source: str | None) -> str:
    if source is not None and f"{oid}@{source}" in record["logical_objects"]:
        return f"{oid}@{source}"
    return oid


def resolve_targets(record: Mapping[str, Any], targets: Any = "all", source: str | None = None) -> list[dict]:
    """Restore plans, one per snapshot that is read:
    ``{"snapshot": index, "path": ..., "objects": {id: size}, "remap": [{"id", "snapshot_range", "object_range",
    "hash", "as": local id}]}``."""
    if isinstance(targets, Mapping):
        plans: list[dict] = []
        for src, ids in targets.items():
            for p in resolve_targets(record, list(ids), source=str(src)):
                p["for_source"] = str(src)
                plans.append(p)
        return plans
    if targets == "all":
        ids: Iterable[str] = list(record["logical_objects"])
    elif hasattr(targets, "initial_objects"):
        ids = list(persisted_objects(targets))
    else:
        ids = list(targets)
    by_snap: dict[int, dict] = {}
    for want in ids:
        oid = _qualified(record, want, source)
        if oid not in record["logical_objects"]:
            raise KeyError(f"checkpoint has no object {want!r}" + (f" for source {source}" if source else ""))
        spans: dict[tuple[int, int], dict] = {}
        for e in record["slices"].get(oid, ()):
            key = (int(e["object_range"][0]), int(e["object_range"][1]))
            if key not in spans or int(e["snapshot"]) < int(spans[key]["snapshot"]):
                spans[key] = e
        for key in sorted(spans):
            e = spans[key]
            si = int(e["snapshot"])
            snap = record["snapshots"][si]
            plan = by_snap.setdefault(si, {"snapshot": si, "path": snap["path"], "objects": {}, "remap": []})
            plan["objects"][oid] = int(record["logical_objects"][oid]["bytes"])
            plan["remap"].append({"id": oid, "as": want, "snapshot_object": e.get("snapshot_object", oid.split("@", 1)[0]),
                                  "snapshot_range": list(e["snapshot_range"]),
                                  "object_range": list(e["object_range"]), "hash": e.get("hash")})
    return [by_snap[k] for k in sorted(by_snap)]
