"""Engine snapshots: selected slices of store objects → files of ≤ 64 MiB chunks plus a manifest
with a blake2b-16 hash per slice (``dataflow-snapshot/v1``).  A snapshot job runs on its own payload
thread under **read leases**; restore is three passes (validate manifest and remap, place
destinations, copy + verify hashes).  Role parity: reference
``src/dataflow/service/handlers_snapshot.py:45-524``."""
from __future__ import annotations

import hashlib
import json
import os
import threading
import time
from pathlib import Path

from .wire import ServiceError

SNAPSHOT_SCHEMA = "dataflow-snapshot/v1"
CHUNK_BYTES = 64 << 20
MANIFEST = "snapshot_manifest.json"


def slice_hash(view) -> str:
    h = hashlib.blake2b(digest_size=16)
    for off in range(0, len(view), CHUNK_BYTES):
        h.update(view[off:off + CHUNK_BYTES])
    return h.hexdigest()


def resolve_slices(store, spec) -> list[dict]:
    """``spec``: list of ids or of ``{"id", "offset", "size", "as"}``; returns concrete slices."""
    out = []
    for s in spec:
        if isinstance(s, str):
            s = {"id": s}
        r = store.get(s["id"])
        off = int(s.get("offset", 0))
        size = int(s.get("size", r.size - off))
        if off < 0 or size < 0 or off + size > r.size:
            raise ServiceError("BAD_REQUEST", f"slice {s} lies outside object {r.id!r} ({r.size} bytes)")
        out.append({"id": r.id, "offset": off, "size": size, "as": s.get("as", r.id), "object_size": r.size})
    return out


def write_snapshot(dest, slices: list[dict], view_of, client_meta=None, progress=None) -> dict:
    """Write ``slices`` (concrete: id / offset / size / as) of the objects ``view_of(id) -> memoryview`` into
    ``dest`` as chunk files plus the manifest (written last).  Usable without a daemon."""
    dest = Path(dest)
    dest.mkdir(parents=True, exist_ok=True)
    entries = []
    for i, s in enumerate(slices):
        view = view_of(s["id"])[s["offset"]:s["offset"] + s["size"]]
        files = []
        for c, off in enumerate(range(0, max(s["size"], 1), CHUNK_BYTES)):
            name = f"slice{i:05d}_{c:04d}.bin"
            with open(dest / name, "wb") as f:
                f.write(view[off:off + CHUNK_BYTES])
            files.append(name)
            if progress is not None:
                progress(len(view[off:off + CHUNK_BYTES]))
        entries.append({**s, "files": files, "hash": slice_hash(view)})
    manifest = {"schema": SNAPSHOT_SCHEMA, "created": time.time(), "slices": entries,
                "client_meta": dict(client_meta or {}), "total_bytes": sum(s["size"] for s in slices)}
    tmp = dest / (MANIFEST + ".tmp")
    tmp.write_text(json.dumps(manifest, indent=1))
    os.replace(tmp, dest / MANIFEST)                 # the manifest lands last: it is the completeness marker
    return manifest


def read_snapshot_slice(path, entry: dict) -> bytes:
    """Bytes of one manifest entry, hash-verified."""
    buf = bytearray()
    for name in entry["files"]:
        try:
            with open(Path(path) / name, "rb") as f:
                buf += f.read()
        except OSError as e:
            raise ServiceError("VERIFY_FAILED", f"slice of {entry['as']!r} in {path}: file {name!r} cannot be read ({type(e).__name__})") from None
    buf = bytes(buf[:entry["size"]])
    if slice_hash(memoryview(buf)) != entry["hash"]:
        raise ServiceError("VERIFY_FAILED", f"slice of {entry['as']!r} in {path} does not match its recorded hash")
    return buf


def snapshot_job(server, job: dict) -> None:
    st = server.store
    ids = sorted({s["id"] for s in job["slices"]})
    try:
        def progress(n):
            job["bytes_done"] += n
        manifest = write_snapshot(job["dest"], job["slices"], st.view, job.get("client_meta", {}), progress)
        job.update(state="done", hashes={e["as"] + f"@{e['offset']}": e["hash"] for e in manifest["slices"]},
                   manifest=manifest)
    except Exception as e:          # noqa: BLE001
        job.update(state="failed", message=f"{type(e).__name__}: {e}")
    finally:
        st.release_leases(ids)
        job["finished"] = time.time()
        server.state.emit("snapshot_" + job["state"], job_id=job["job_id"])


def read_manifest(path) -> dict:
    p = Path(path) / MANIFEST
    if not p.exists():
        raise ServiceError("UNKNOWN_SNAPSHOT", f"no complete snapshot at {path}")
    try:
        m = json.loads(p.read_text())
    except (ValueError, OSError) as e:
        raise ServiceError("VERIFY_FAILED", f"the manifest of the snapshot at {path} is damaged ({type(e).__name__}: {e})") from None
    if not isinstance(m, dict) or m.get("schema") != SNAPSHOT_SCHEMA:
        m = m if isinstance(m, dict) else {}
        raise ServiceError("VERSION_SKEW", f"snapshot schema {m.get('schema')!r}, expected {SNAPSHOT_SCHEMA!r}")
    return m


def validate_remap(manifest: dict, remap) -> list[dict]:
    """``remap``: None (restore everything under the saved names) or a list of
    ``{"from": saved name, "from_offset", "size", "to": object id, "to_offset", "to_size"}`` windows."""
    saved = {}
    for e in manifest["slices"]:
        saved.setdefault(e["as"], []).append(e)
    plan = []
    if remap is None:
        for e in manifest["slices"]:
            plan.append({"entry": e, "src_off": 0, "size": e["size"], "to": e["as"], "to_offset": e["offset"],
                         "to_size": e["object_size"]})
        return plan
    for w in remap:
        name = w["from"]
        if name not in saved:
            raise ServiceError("UNKNOWN_OBJECT", f"snapshot holds no object {name!r}")
        fo, size = int(w.get("from_offset", 0)), int(w["size"])
        e = next((x for x in saved[name] if x["offset"] <= fo and fo + size <= x["offset"] + x["size"]), None)
        if e is None:
            raise ServiceError("BAD_REQUEST", f"window {w} is not covered by one saved slice of {name!r}")
        plan.append({"entry": e, "src_off": fo - e["offset"], "size": size, "to": w.get("to", name),
                     "to_offset": int(w.get("to_offset", fo)), "to_size": int(w.get("to_size", e["object_size"]))})
    return plan


def restore_job(server, job: dict) -> None:
    st = server.store
    src = Path(job["path"])
    try:
        plan = job["plan"]
        # pass 2: place destinations
        for w in plan:
            r = st.objects.get(w["to"])
            if r is None:
                st.create(w["to"], w["to_size"])
            elif r.size != w["to_size"]:
                raise ServiceError("BINDING_MISMATCH", f"{w['to']!r} is {r.size} bytes, snapshot wants {w['to_size']}")
        # pass 3: copy and verify
        verified: dict[int, bool] = {}
        for w in plan:
            e = w["entry"]
            buf = bytearray()
            for name in e["files"]:
                try:
                    buf += (src / name).read_bytes()
                except OSError as err:
                    raise ServiceError("VERIFY_FAILED", f"slice of {e['as']!r}: file {name!r} cannot be read ({type(err).__name__})") from None
            if id(e) not in verified:
                if slice_hash(memoryview(buf)) != e["hash"]:
                    raise ServiceError("VERIFY_FAILED", f"slice of {e['as']!r} does not match its recorded hash")
                verified[id(e)] = True
            st.view(w["to"])[w["to_offset"]:w["to_offset"] + w["size"]] = buf[w["src_off"]:w["src_off"] + w["size"]]
            job["bytes_done"] += w["size"]
        job.update(state="done")
    except ServiceError as e:
        job.update(state="failed", message=str(e), code=e.code)
    except Exception as e:          # noqa: BLE001
        job.update(state="failed", message=f"{type(e).__name__}: {e}", code="IO_ERROR")
    finally:
        job["finished"] = time.time()
        server.state.emit("restore_" + job["state"], job_id=job["job_id"])


def install(server) -> None:
    H, st = server.handlers, server.store

    def snapshot(req, payload):
        slices = resolve_slices(st, req.get("slices") or [r.id for r in st.objects.values()])
        ids = sorted({s["id"] for s in slices})
        st.acquire_leases(ids)
        job = {"job_id": server.state.new_id("s"), "kind": "snapshot", "state": "running", "dest": req["dest"],
               "slices": slices, "client_meta": req.get("client_meta", {}), "bytes_done": 0, "started": time.time()}
        server.jobs[job["job_id"]] = job
        threading.Thread(target=snapshot_job, args=(server, job), name="dataflowd-snapshot", daemon=True).start()
        return {"job_id": job["job_id"], "slices": len(slices)}
    H["snapshot"] = snapshot

    def status(kind, err):
        def h(req, payload):
            job = server.jobs.get(req["job_id"])
            if job is None or job["kind"] != kind:
                raise ServiceError(err, req["job_id"])
            return {k: v for k, v in job.items() if k not in ("slices", "plan", "manifest")}
        return h
    H["snapshot_status"] = status("snapshot", "UNKNOWN_SNAPSHOT")
    H["restore_status"] = status("restore", "UNKNOWN_RESTORE")

    def restore_snapshot(req, payload):
        manifest = read_manifest(req["path"])                      # pass 1: validate
        plan = validate_remap(manifest, req.get("remap"))
        job = {"job_id": server.state.new_id("t"), "kind": "restore", "state": "running", "path": req["path"],
               "plan": plan, "bytes_done": 0, "started": time.time()}
        server.jobs[job["job_id"]] = job
        if req.get("sync", True):
            restore_job(server, job)                               # on the dispatcher: ordered with runs
        else:
            threading.Thread(target=restore_job, args=(server, job), name="dataflowd-restore", daemon=True).start()
        return {"job_id": job["job_id"], "state": job["state"], "message": job.get("message", "")}
    H["restore_snapshot"] = restore_snapshot
