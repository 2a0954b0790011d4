"""Training checkpoints: ``<dir>/step_{n:06d}/`` holds one engine snapshot per rank (``rank{i}/``), the exact
lowered programs (``programs/rank{i}.json``) and the checkpoint record, which is written last.

``save_checkpoint(trainer, ...)`` works for a solo trainer and, when ``torch.distributed`` is initialised, for
every rank of a job calling it at the same step: each rank snapshots its own persistent objects, rank 0 gathers
the slice hashes and writes the record.  Sharded weights (``Ws_*``) are recorded as byte ranges of the logical
``W_*`` object, so a checkpoint taken at one world size restores its weights at another; sharded optimizer state is
recorded as spans of logical planes (``O_3.master``, ``O_3.m``, ``O_3.v``: one plane per state field of the whole
parameter), so it restores at another world size too.  ``load_checkpoint`` reads the record,
verifies every slice hash, fills the host store and drops device-resident copies; the returned payload carries
the losses and the data cursor, so a resumed curve continues exactly.
Role parity: reference ``src/dataflow_training/run/checkpointing.py:25-420``.
"""
from __future__ import annotations

import json
import os
import re
import shutil
from typing import Any, Mapping

from ..checkpoint import read_record, resolve_targets, save_checkpoint as compose_checkpoint
from ..checkpoint.compose import SourceSlice
from ..checkpoint.record import has_record
from ..core.jsonio import save_program
from ..service.snapshots import read_manifest, read_snapshot_slice, resolve_slices, write_snapshot  # noqa: F401

STEP_DIR = re.compile(r"^step_(\d{6,})$")


def step_dir(root: str, step: int) -> str:
    return os.path.join(root, f"step_{int(step):06d}")


def list_checkpoints(root: str) -> list[tuple[int, str]]:
    out = []
    if os.path.isdir(root):
        for name in os.listdir(root):
            m = STEP_DIR.match(name)
            if m and has_record(os.path.join(root, name)):
                out.append((int(m.group(1)), os.path.join(root, name)))
    return sorted(out)


def resolve_resume(spec: str | None, root: str | None = None) -> str | None:
    """``None`` / ``"none"`` -> no resume; ``"latest"`` -> newest complete step under ``root``; else a step
    directory (or a root, meaning its latest).  Directories without a record are never resumable."""
    if not spec or spec == "none":
        return None
    if spec == "latest":
        found = list_checkpoints(root or "")
        return found[-1][1] if found else None
    if has_record(spec):
        return spec
    found = list_checkpoints(spec)
    if found:
        return found[-1][1]
    raise FileNotFoundError(f"{spec}: no complete checkpoint (no checkpoint_record.json)")


def _world(trainer) -> tuple[int, int]:
    z = trainer.zero or {}
    if z:
        return int(z.get("rank", 0)), int(z.get("world", 1))
    groups = getattr(trainer, "groups", None) or {}
    for inner in ("tp", "ep"):                     # a dp x tp / dp x ep mesh: consecutive ranks form the inner group
        if inner in groups and "dp" in groups:
            g, dp = groups[inner], groups["dp"]
            return int(dp.rank) * int(g.world) + int(g.rank), int(dp.world) * int(g.world)
    for key in ("tp", "ep", "dp"):                 # tensor / expert parallel jobs and plain replicas: the group knows the rank
        g = groups.get(key)
        if g is not None:
            return int(g.rank), int(g.world)
    return 0, 1


def _private_scheme(trainer) -> str | None:
    """``tp`` / ``ep``: every rank's persistent objects are its own cut of the model (or its own replica): they are
    recorded per rank and a resume needs the same scheme and world size."""
    md = trainer.program.metadata or {}
    if int(md.get("tp", 1)) > 1:
        return "tp"
    if int(md.get("ep", 1)) > 1:
        return "ep"
    return None


class TrainerSource:
    """The persistent objects of one in-process trainer as a checkpoint source."""

    def __init__(self, trainer):
        self.t = trainer
        self.rank, self.world = _world(trainer)
        self.name = str(self.rank)
        self._pending: dict[int, dict] = {}

    def persistent(self) -> dict[str, int]:
        return {o.id: int(o.size_bytes) for o in self.t.program.initial_objects if o.persistent}

    def logical_objects(self) -> dict[str, int]:
        out: dict[str, int] = {}
        for s in self.slices():
            out[s.logical_id] = max(out.get(s.logical_id, 0), s.logical_offset + s.size)
        meta = (self.t.program.metadata or {}).get("zero_full_bytes") or {}
        for k, v in meta.items():
            if k in out:
                out[k] = int(v)
        return out

    def slices(self) -> list[SourceSlice]:
        out = []
        full = (self.t.program.metadata or {}).get("zero_full_bytes") or {}
        private = _private_scheme(self.t) if self.world > 1 else None
        for oid, size in self.persistent().items():
            if private:
                out.append(SourceSlice(oid, 0, size, f"{oid}@{self.rank}", 0))
            elif oid.startswith("Ws_") and self.world > 1:
                logical = "W_" + oid[3:]
                total = int(full.get(logical, size * self.world))
                lo = min(size * self.rank, total)
                n = max(min(size, total - lo), 0)
                if n:
                    out.append(SourceSlice(oid, 0, n, logical, lo))
            elif self.world > 1 and oid.startswith("O_") and (self.t.zero or {}).get("stage"):
                out += self._optimizer_planes(oid, size, full)
            else:
                out.append(SourceSlice(oid, 0, size, oid, 0))
        return out

    def _optimizer_planes(self, oid: str, size: int, full: Mapping[str, int]) -> list[SourceSlice]:
        """A rank's sharded optimizer state as spans of LOGICAL planes: ``O_3.m`` is the first-moment plane of the whole
        ``W_3``, and this rank holds the elements of its slice of the parameter.  Recorded this way the state restores
        at any world size (every rank of the new job reads the spans that cover its new slice).  State that does not
        follow a plane layout this function knows is recorded per rank, as before."""
        from ..parallel.zero import slice_bytes, slice_range, split_opt_layout, zero_opt_layout
        name = oid[2:]
        sizes = self.persistent()
        total = int(full.get("W_" + name) or sizes.get("W_" + name) or 0)
        if not total:
            return [SourceSlice(oid, 0, size, f"{oid}@{self.rank}", 0)]
        per = slice_bytes(total, self.world)
        regather = bool((self.t.zero or {}).get("regather"))
        lay = split_opt_layout(per) if (regather and name.isdigit()) else zero_opt_layout(per)
        if lay.size_bytes != size:
            return [SourceSlice(oid, 0, size, f"{oid}@{self.rank}", 0)]
        lo, ln = slice_range(total, self.world, self.rank)           # bytes of the bf16 parameter
        offs = lay.offsets()
        out = []
        for f in lay.fields:
            eb = f.nbytes // max(per // 2, 1)                         # bytes per element of this plane
            if ln:
                out.append(SourceSlice(oid, offs[f.name], (ln // 2) * eb, f"{oid}.{f.name}", (lo // 2) * eb))
        return out

    def write_slices(self, redundancy: int | None = None) -> list[SourceSlice]:
        """What this rank writes at a save.  Objects every rank holds in full (replicas: their logical id is the object
        id) are written by the first ``redundancy`` ranks only; ``None`` = by every rank, which lets the composer check
        all replicas against each other for drift."""
        out = self.slices()
        if redundancy and self.world > 1 and self.rank >= int(redundancy):
            out = [s for s in out if s.logical_id != s.object_id]
        return out

    def resident_objects(self) -> dict[str, int]:
        return self.persistent()

    def start_snapshot(self, dest: str, slices: list[dict], client_meta: Mapping[str, Any]):
        self.t.sync_to_host()
        store = self.t.store
        concrete = [{"id": s["id"], "offset": int(s["offset"]), "size": int(s["size"]), "as": s["id"],
                     "object_size": store.sizes[s["id"]]} for s in slices]

        def view_of(oid):
            import ctypes
            b = store.buffer(oid)
            return memoryview((ctypes.c_char * b.size).from_address(b.ptr)).cast("B")
        manifest = write_snapshot(dest, concrete, view_of, client_meta)
        return manifest

    def wait_snapshot(self, handle, timeout):
        return handle

    def engine_spec(self) -> dict:
        return {"backing_bytes": int(self.t.store.total), "device": self.t.device,
                "kernel_set": sorted(set(self.t.K.describe().values())), "fake": False}


def save_checkpoint(trainer, root: str, step: int, *, seed: int = 0, client_payload: Any = None, summary: Any = None,
                    launch: Any = None, keep_last: int | None = None, scheme: Mapping[str, Any] | None = None,
                    redundancy: int | None = None) -> str:
    """Every rank of the job calls this at the same step.  Returns the step directory.  ``redundancy``: how many ranks
    write their copy of the replicated objects (default: all of them)."""
    src = TrainerSource(trainer)
    sdir = step_dir(root, step)
    rank, world = src.rank, src.world
    os.makedirs(os.path.join(sdir, "programs"), exist_ok=True)
    save_program(trainer.program, os.path.join(sdir, "programs", f"rank{rank}.json"))
    if world == 1:
        compose_checkpoint([src], sdir, step=step, seed=seed, logical_objects=src.logical_objects(),
                           scheme={"world": 1, **dict(scheme or {})}, client_payload=client_payload, summary=summary,
                           launch=launch)
    else:
        import torch.distributed as dist
        wr = src.write_slices(redundancy)
        manifest = src.start_snapshot(os.path.join(sdir, f"rank{rank}"),
                                      [{"id": s.object_id, "offset": s.offset, "size": s.size} for s in wr],
                                      {"step": step, "source": src.name})
        mine = {"name": src.name, "slices": [vars(s) for s in wr], "resident": src.resident_objects(),
                "hashes": {f"{e['as']}@{e['offset']}": e["hash"] for e in manifest["slices"]}, "spec": src.engine_spec(),
                "logical": src.logical_objects()}
        gathered: list[Any] = [None] * world
        dist.all_gather_object(gathered, mine)
        if rank == 0:
            sources = [_Recorded(g) for g in gathered]
            logical: dict[str, int] = {}
            for g in gathered:
                for k, v in g["logical"].items():
                    logical[k] = max(logical.get(k, 0), int(v))
            compose_checkpoint(sources, sdir, step=step, seed=seed, logical_objects=logical,
                               scheme={"world": world, "zero": trainer.zero, "parallel": _private_scheme(trainer),
                                       "replica_copies": min(int(redundancy), world) if redundancy else world, **dict(scheme or {})},
                               client_payload=client_payload, summary=summary, launch=launch)
        dist.barrier()
    if keep_last and rank == 0:
        for _, old in list_checkpoints(root)[:-int(keep_last)]:
            shutil.rmtree(old, ignore_errors=True)
    return sdir


class _Recorded:
    """A rank whose snapshot is already on disk (its facts were gathered to the composing rank)."""

    def __init__(self, g: Mapping[str, Any]):
        self.g = g
        self.name = g["name"]

    def slices(self):
        return [SourceSlice(**s) for s in self.g["slices"]]

    def resident_objects(self):
        return dict(self.g["resident"])

    def start_snapshot(self, dest, slices, client_meta):
        return None

    def wait_snapshot(self, handle, timeout):
        return {"slices": [{"as": k.rsplit("@", 1)[0], "offset": int(k.rsplit("@", 1)[1]), "hash": h}
                           for k, h in self.g["hashes"].items()]}

    def engine_spec(self):
        return dict(self.g["spec"])


def load_checkpoint(trainer, sdir: str, only_prefixes: tuple[str, ...] | None = None) -> dict:
    """Fill the trainer's host store from a step directory; returns the record (``client_payload`` has the
    caller's resume state).  Device-resident copies are dropped so the next step reloads from the store.
    ``only_prefixes``: restore only objects whose id starts with one of these (``("W_",)``: the weights alone, which
    is what an evaluation needs and what restores across world sizes and optimizer-sharding modes)."""
    import ctypes
    rec = read_record(sdir)
    src = TrainerSource(trainer)
    want = [s for s in src.slices() if only_prefixes is None or s.object_id.startswith(tuple(only_prefixes))]
    store = trainer.store
    for s in want:                                   # an object may be several spans (the planes of sharded optimizer state)
        oid = s.object_id
        logical = s.logical_id
        if logical not in rec["logical_objects"]:
            raise KeyError(f"checkpoint {sdir} has no object {logical!r} (needed for {oid!r} of rank {src.rank})")
        lo, hi = s.logical_offset, s.logical_offset + s.size
        filled = 0
        spans: dict[tuple[int, int], dict] = {}
        for e in rec["slices"][logical]:
            key = (int(e["object_range"][0]), int(e["object_range"][1]))
            if key not in spans or int(e["snapshot"]) < int(spans[key]["snapshot"]):
                spans[key] = e
        for (a, b), e in sorted(spans.items()):
            if b <= lo or a >= hi:
                continue
            snap = rec["snapshots"][int(e["snapshot"])]
            manifest = read_manifest(os.path.join(sdir, snap["path"]))
            local = e.get("snapshot_object", logical)
            ent = next(m for m in manifest["slices"] if m["as"] == local and int(m["offset"]) == int(e["snapshot_range"][0]))
            data = read_snapshot_slice(os.path.join(sdir, snap["path"]), ent)
            ca, cb = max(a, lo), min(b, hi)
            dst = store.buffer(oid).ptr + s.offset + (ca - lo)
            ctypes.memmove(dst, data[ca - a:cb - a], cb - ca)
            filled += cb - ca
        if filled != s.size:
            raise ValueError(f"{oid}: checkpoint covers {filled} of the {s.size} bytes this rank needs")
    trainer.session.drop_resident()
    trainer.step_index = int(rec["step"])
    return rec


def peek(sdir: str) -> dict:
    """Display facts of a checkpoint without touching its payload."""
    rec = read_record(sdir)
    return {"step": rec["step"], "seed": rec["seed"], "scheme": rec["scheme"], "summary": rec.get("summary"),
            "objects": len(rec["logical_objects"]), "bytes": sum(int(v["bytes"]) for v in rec["logical_objects"].values()),
            "snapshots": [s["path"] for s in rec["snapshots"]], "launch": (rec.get("launch") or {}).get("argv")}
