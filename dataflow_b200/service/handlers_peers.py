"""Peer verbs of the engine service: links, object sends, groups, bench verbs.
Role parity: reference ``src/dataflow/service/handlers_peers.py:57-339``."""
from __future__ import annotations

import time

import numpy as np

from .wire import ServiceError


def install(server) -> None:
    nm = server.nm
    H = server.handlers

    def need_nm():
        if nm is None:
            raise ServiceError("PEER_DISABLED", "this daemon was started without --peer-name")

    def peer_connect(req, payload):
        need_nm()
        return nm.connect(req.get("name") or req["peer"], req.get("address") or req["addr"], float(req.get("timeout", 10.0)))

    def peer_disconnect(req, payload):
        need_nm()
        nm.disconnect(req.get("name") or req["peer"])
        return {}

    def send_object(req, payload):
        need_nm()
        server.store.get(req["id"])
        xid = nm.send_object(req["peer"], req["id"], req.get("as_id") or req.get("dest"))
        if req.get("wait", True):
            st = nm.wait_transfer(xid, float(req.get("timeout", 600.0)))
            if st["state"] != "COMPLETE":
                raise ServiceError("IO_ERROR", f"send of {req['id']!r} to {req['peer']!r} ended {st['state']}: {st.get('error', '')}", transfer=st)
            return {"transfer_id": xid, "state": "done", "transfer": st}
        return {"transfer_id": xid, "state": "running"}

    def transfer_status(req, payload):
        need_nm()
        st = nm.transfer_status(req.get("transfer_id") or req["xid"])
        state = {"COMPLETE": "done", "FAILED": "failed", "UNKNOWN": "failed"}.get(st["state"], "running")
        return {"state": state, "message": st.get("error", ""), "transfer": st}

    def create_peer_group(req, payload):
        need_nm()
        backend = nm.resolve_backend(req.get("backend", "auto"), server.config.fake or server.config.device is None)
        return nm.create_group(req["name"], list(req["members"]), backend, float(req.get("timeout", 30.0)))

    def destroy_peer_group(req, payload):
        need_nm()
        nm.destroy_group(req["name"])
        return {}

    def list_peer_groups(req, payload):
        need_nm()
        return {"groups": nm.groups.list()}

    def list_peers(req, payload):
        need_nm()
        return {"peers": nm.list_peers(), "name": nm.name, "port": nm.port}

    def peer_status(req, payload):
        need_nm()
        who = req.get("name") or req["peer"]
        hits = [p for p in nm.list_peers() if p["peer"] == who]
        if not hits:
            raise ServiceError("PEER_UNREACHABLE", f"no link to peer {who!r}")
        return {"peer": hits[0], "core": dict(nm.core.stats)}

    def p2p_bench(req, payload):
        need_nm()
        return nm.bw_probe(req["peer"], max(int(req.get("nbytes", 64 << 20)) >> 20, 1))

    def coll_bench(req, payload):
        """All-reduce of a seeded vector over a group, with a correctness check against the closed form."""
        need_nm()
        g = nm.groups.get(req["group"])
        n = max(int(req.get("nbytes", 1 << 18)) // 4, 1)
        rank = g.rank_of(nm.name)
        x = np.full(n, float(rank + 1), dtype=np.float32)
        t0 = time.perf_counter()
        y = nm.all_reduce(req["group"], x, float(req.get("timeout", 60.0)))
        dt = time.perf_counter() - t0
        want = float(sum(range(1, len(g.members) + 1)))
        return {"ok": bool(np.all(y == want)), "seconds": dt, "bytes": int(x.nbytes), "expected": want, "got": float(y[0])}

    def debug_sever(req, payload):
        need_nm()
        nm.debug_sever(req["peer"])
        return {}

    H.update({"peer_connect": peer_connect, "peer_disconnect": peer_disconnect, "send_object": send_object,
              "transfer_status": transfer_status, "create_peer_group": create_peer_group,
              "destroy_peer_group": destroy_peer_group, "list_peer_groups": list_peer_groups, "list_peers": list_peers,
              "peer_status": peer_status, "p2p_bench": p2p_bench, "coll_bench": coll_bench,
              "debug_sever": debug_sever})
