"""EngineClient: one method per service verb, payload streaming, waits for snapshot / restore jobs.
Verb set parity: reference ``src/dataflow/service/client.py:175-455``."""
from __future__ import annotations

import socket
import time
from typing import Any, Mapping

from ..core import Program, program_to_dict
from .wire import SCHEMA_VERSION, Conn, ServiceError


class EngineClient:
    def __init__(self, socket_path: str, client_name: str = "client", timeout: float | None = None):
        s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        if timeout:
            s.settimeout(timeout)
        s.connect(socket_path)
        self.conn = Conn(s)
        self.conn.send({"schema": SCHEMA_VERSION, "client": client_name})
        hello, _ = self.conn.recv()
        if hello is None or not hello.get("ok"):
            err = (hello or {}).get("error", {})
            raise ServiceError(err.get("code", "INTERNAL"), err.get("message", "handshake failed"))
        self.server_info = hello

    def call(self, op: str, payload: bytes | memoryview | None = None, **fields: Any):
        self.conn.send({"op": op, **fields}, payload)
        rep, data = self.conn.recv()
        if rep is None:
            raise ConnectionError("daemon closed the connection")
        if not rep.get("ok"):
            e = rep.get("error", {})
            raise ServiceError(e.pop("code", "INTERNAL"), e.pop("message", ""), **e)
        return (rep, data) if data is not None else rep

    def close(self) -> None:
        self.conn.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- status
    def health(self): return self.call("health")
    def engine_status(self): return self.call("engine_status")
    def session_status(self): return self.call("session_status")
    def subscribe_events(self, since: int = 0): return self.call("subscribe_events", since=since)["events"]
    def shutdown(self): return self.call("shutdown")

    # -- store
    def put_object(self, oid: str, data) -> dict: return self.call("put_object", data, id=oid)
    def get_object(self, oid: str, offset: int = 0, size: int | None = None) -> bytes:
        f = {"id": oid, "offset": offset}
        if size is not None:
            f["size"] = size
        rep = self.call("get_object", **f)
        return rep[1] if isinstance(rep, tuple) else b""
    def create_object(self, oid: str, size: int, replace: bool = False): return self.call("create_object", id=oid, size=size, replace=replace)
    def materialize_object(self, oid: str, size: int, kind: str = "zeros", **kw): return self.call("materialize_object", id=oid, size=size, kind=kind, **kw)
    def release_object(self, oid: str): return self.call("release_object", id=oid)
    def protect_object(self, oid: str): return self.call("protect_object", id=oid)
    def unprotect_object(self, oid: str): return self.call("unprotect_object", id=oid)
    def duplicate_object(self, src: str, dst: str): return self.call("duplicate_object", src=src, dst=dst)
    def wipe(self, scope: str = "unprotected", force: bool = False): return self.call("wipe", scope=scope, force=force)
    def query_object(self, oid: str): return self.call("query_object", id=oid)
    def list_objects(self): return self.call("list_objects")["objects"]
    def query_backing(self): return self.call("query_backing")
    def query_fast(self): return self.call("query_fast")

    # -- snapshots
    def snapshot(self, dest: str, slices=None, client_meta: Mapping | None = None):
        return self.call("snapshot", dest=dest, slices=slices, client_meta=dict(client_meta or {}))
    def snapshot_status(self, job_id: str): return self.call("snapshot_status", job_id=job_id)
    def restore_snapshot(self, path: str, remap=None, sync: bool = True): return self.call("restore_snapshot", path=path, remap=remap, sync=sync)
    def restore_status(self, job_id: str): return self.call("restore_status", job_id=job_id)

    def _wait(self, fn, job_id: str, timeout: float):
        t0 = time.time()
        while True:
            s = fn(job_id)
            if s["state"] != "running":
                if s["state"] != "done":
                    raise ServiceError(s.get("code", "IO_ERROR"), s.get("message", "job failed"))
                return s
            if time.time() - t0 > timeout:
                raise TimeoutError(f"job {job_id} still running after {timeout}s")
            time.sleep(0.01)

    def wait_snapshot(self, job_id: str, timeout: float = 600.0): return self._wait(self.snapshot_status, job_id, timeout)
    def wait_restore(self, job_id: str, timeout: float = 600.0): return self._wait(self.restore_status, job_id, timeout)

    # -- programs and runs
    def register_program(self, program: Program | dict, resolver_spec: Mapping | None = None, expect_prog_id: str | None = None,
                         prepare_placement: bool = False, placement_capacity: int | None = None):
        """``prepare_placement``: the daemon also computes a static placement of the program's fast allocations by a dry run
        (refused when none fits ``placement_capacity`` / the program's own capacity) and uses it for its runs."""
        d = program if isinstance(program, dict) else program_to_dict(program)
        return self.call("register_program", program=d, resolver_spec=dict(resolver_spec) if resolver_spec else None,
                         expect_prog_id=expect_prog_id, prepare_placement=bool(prepare_placement), placement_capacity=placement_capacity)
    def validate_program(self, program: Program | dict):
        return self.call("validate_program", program=program if isinstance(program, dict) else program_to_dict(program))
    def unregister_program(self, prog_id: str): return self.call("unregister_program", prog_id=prog_id)
    def load_plugin(self, module: str): return self.call("load_plugin", module=module)
    def run(self, prog_id: str, args: Mapping | None = None, fetch=None, trace: bool = False):
        return self.call("run", prog_id=prog_id, args=dict(args or {}), fetch=list(fetch or ()), trace=trace)
    def cancel_run(self, run_id: str = ""): return self.call("cancel_run", run_id=run_id)
    def run_status(self, run_id: str): return self.call("run_status", run_id=run_id)
    def list_runs(self): return self.call("list_runs")["runs"]
    def run_events(self, since: int = 0): return self.call("run_events", since=since)["events"]
    def export_trace(self, run_id: str): return self.call("export_trace", run_id=run_id)["trace"]
    def list_programs(self): return self.call("list_programs")["programs"]
    def list_resolvers(self): return self.call("list_resolvers")["resolvers"]

    # -- peers
    def peer_connect(self, name: str, address: str): return self.call("peer_connect", name=name, address=address)
    def peer_disconnect(self, name: str): return self.call("peer_disconnect", name=name)
    def list_peers(self): return self.call("list_peers")["peers"]
    def peer_status(self, name: str): return self.call("peer_status", name=name)
    def send_object(self, peer: str, oid: str, as_id: str | None = None): return self.call("send_object", peer=peer, id=oid, as_id=as_id or oid)
    def transfer_status(self, transfer_id: str): return self.call("transfer_status", transfer_id=transfer_id)
    def wait_transfer(self, transfer_id: str, timeout: float = 120.0):
        t0 = time.time()
        while True:
            s = self.transfer_status(transfer_id)
            if s["state"] in ("done", "failed"):
                if s["state"] == "failed":
                    raise ServiceError("PEER_UNREACHABLE", s.get("message", "transfer failed"))
                return s
            if time.time() - t0 > timeout:
                raise TimeoutError(transfer_id)
            time.sleep(0.01)
    def create_peer_group(self, name: str, members, backend: str = "auto", timeout: float = 30.0):
        return self.call("create_peer_group", name=name, members=list(members), backend=backend, timeout=timeout)
    def destroy_peer_group(self, name: str): return self.call("destroy_peer_group", name=name)
    def list_peer_groups(self): return self.call("list_peer_groups")["groups"]
    def p2p_bench(self, peer: str, nbytes: int = 1 << 24): return self.call("p2p_bench", peer=peer, nbytes=nbytes)
    def coll_bench(self, group: str, op: str = "allreduce", nbytes: int = 1 << 20): return self.call("coll_bench", group=group, coll_op=op, nbytes=nbytes)
    def profiler_control(self, action: str): return self.call("profiler_control", action=action)
