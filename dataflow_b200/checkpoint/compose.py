"""``save_checkpoint``: fan one engine snapshot out per source, wait for all of them, collect the per-slice
hashes, check replicas for drift, and write the record last.

A *source* is anything that holds checkpointable bytes and can snapshot slices of them: an ``EngineClient``
wrapped by ``ClientSource`` (one daemon per rank), or an in-process holder (``run.checkpointing.TrainerSource``).
Each source declares which logical byte ranges its objects cover (``SourceSlice``).
Contract parity: reference ``src/dataflow/checkpoint/compose.py:30-160``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Mapping, Protocol

from .record import RecordError, build_record, write_record


@dataclass
class SourceSlice:
    object_id: str                      # the source's local object
    offset: int                         # byte range inside the local object
    size: int
    logical_id: str                     # the record's name (may be source-qualified: ``Aux_0@1``)
    logical_offset: int                 # where those bytes sit in the logical object


class Source(Protocol):
    name: str

    def slices(self) -> list[SourceSlice]: ...
    def resident_objects(self) -> dict[str, int]: ...
    def start_snapshot(self, dest: str, slices: list[dict], client_meta: Mapping[str, Any]) -> Any: ...
    def wait_snapshot(self, handle: Any, timeout: float) -> dict: ...       # -> manifest
    def engine_spec(self) -> dict: ...


@dataclass
class ClientSource:
    """A dataflowd rank behind an ``EngineClient``."""
    name: str
    client: Any
    declared: list[SourceSlice] = field(default_factory=list)

    def slices(self):
        return self.declared

    def resident_objects(self):
        want = {s.object_id for s in self.declared}
        return {o["id"]: int(o["size"]) for o in self.client.list_objects() if o["id"] in want}

    def start_snapshot(self, dest, slices, client_meta):
        return self.client.snapshot(dest, slices=slices, client_meta=client_meta)["job_id"]

    def wait_snapshot(self, handle, timeout):
        job = self.client.wait_snapshot(handle, timeout)
        return {"slices": [{"as": k.rsplit("@", 1)[0], "offset": int(k.rsplit("@", 1)[1]), "hash": h}
                           for k, h in job["hashes"].items()]}

    def engine_spec(self):
        st = self.client.engine_status()
        return {k: st.get(k) for k in ("backing_bytes", "device", "kernel_set", "fake") if k in st}


def save_checkpoint(sources: list[Source], step_dir: str, *, step: int, seed: int = 0,
                    logical_objects: Mapping[str, int], scheme: Mapping[str, Any] | None = None,
                    client_payload: Any = None, summary: Any = None, launch: Any = None,
                    timeout: float = 3600.0) -> dict:
    """Returns the written record.  ``logical_objects``: ``{logical id: bytes}`` — the namespace that must be
    covered completely by the sources' slices."""
    os.makedirs(step_dir, exist_ok=True)
    handles = []
    for i, src in enumerate(sources):
        sl = [{"id": s.object_id, "offset": s.offset, "size": s.size} for s in src.slices()]
        rel = f"rank{src.name}" if not str(src.name).startswith("rank") else str(src.name)
        handles.append((src, rel, src.start_snapshot(os.path.join(step_dir, rel), sl, {"step": step, "source": src.name})))
    snapshots, slices = [], {}
    for i, (src, rel, h) in enumerate(handles):
        manifest = src.wait_snapshot(h, timeout)
        by_key = {(e["as"], int(e["offset"])): e["hash"] for e in manifest["slices"]}
        snapshots.append({"path": rel, "source": str(src.name), "objects": src.resident_objects()})
        # snapshot byte offsets: the slices of one object are laid out at their own offsets in that object
        for s in src.slices():
            hsh = by_key.get((s.object_id, s.offset))
            if hsh is None:
                raise RecordError(f"source {src.name}: snapshot returned no hash for {s.object_id}@{s.offset}")
            slices.setdefault(s.logical_id, []).append({
                "snapshot": i, "snapshot_object": s.object_id, "snapshot_range": [s.offset, s.offset + s.size],
                "object_range": [s.logical_offset, s.logical_offset + s.size], "hash": hsh})
    rec = build_record(step=step, seed=seed, scheme=scheme or {},
                       logical_objects={k: {"bytes": int(v)} for k, v in logical_objects.items()},
                       snapshots=snapshots, slices=slices,
                       engine_spec={str(src.name): src.engine_spec() for src in sources},
                       client_payload=client_payload, summary=summary, launch=launch)
    write_record(step_dir, rec)
    return rec
