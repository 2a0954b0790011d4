"""NetworkManager: the daemon's links to other daemons.

TCP links carry the framed peer protocol (``wire.Conn``: one JSON line + optional raw payload).  Per link: a HELLO
exchange, a reader thread, PING/PONG heartbeats (every 2 s; a link silent for 6 s is declared down, its open
transfers fail and its groups go to ERROR).  Object sends run through the transport-free ``PeerCore``; chunks land
directly in reserved store extents.  Groups are a star around their coordinator: ``create_group`` sends GROUP_JOIN
down each link and waits for every GROUP_ACK (an attachment barrier).  The ``hostmem`` collective lane reduces
through the coordinator in rank order (deterministic); the ``nccl`` lane hands the group to ``peer.ncclcomm``.
``debug_sever`` closes a link from the host side (fault injection for tests).
Role parity: reference ``src/dataflow/service/peer/nm.py:128-1087``.
"""
from __future__ import annotations

import socket
import threading
import time
from typing import Any

import numpy as np

from ..wire import Conn, ServiceError
from . import protocol as P
from .core import CollectiveQueue, PeerCore
from .groups import GroupTable


class Link:
    def __init__(self, peer: str, conn: Conn, outbound: bool):
        self.peer, self.conn, self.outbound = peer, conn, outbound
        self.send_lock = threading.Lock()
        self.last_heard = time.monotonic()
        self.up = True
        self.bytes_out = 0
        self.bytes_in = 0

    def send(self, frame: dict, payload=None) -> None:
        with self.send_lock:
            self.conn.send(frame, payload)
            self.bytes_out += 0 if payload is None else len(payload)


class HostGroupHandle:
    """What a task sees of a peer group on the ``hostmem`` lane (``ctx.groups[name]``): SUM collectives over the peer plane's
    TCP links.  Tensors on a device are staged through host memory around the exchange, which synchronises the calling
    stream — this is the plumbing lane for CPU ranks and for tests, the counterpart of the reference's hostmem lane
    (``src/dataflow/service/peer/comm.py:139-603``), not a fast path.  Role: ``src/dataflow/runtime/groups.py:22-63``."""

    def __init__(self, nm: "NetworkManager", name: str, timeout: float = 120.0):
        self.nm, self.name, self.timeout = nm, name, timeout
        g = nm.groups.get(name)
        self.rank, self.world, self.lane = g.rank_of(nm.name), len(g.members), "collective"

    def _exchange(self, t):
        import torch
        host = t.detach()
        if host.is_cuda:
            torch.cuda.current_stream(host.device).synchronize()
            host = host.cpu()
        wide = host.float() if host.dtype in (torch.bfloat16, torch.float16) else host
        out = self.nm.all_reduce(self.name, np.ascontiguousarray(wide.contiguous().numpy()), self.timeout)
        return torch.from_numpy(out).to(t.dtype)

    def all_reduce(self, t):
        if self.world > 1:
            t.copy_(self._exchange(t).reshape(t.shape))
        return t

    allreduce = all_reduce

    def reduce_scatter(self, full, out):
        """``out`` receives this rank's ``1 / world`` slice of the sum of ``full`` (sum first, slice after: the lane is for
        correctness, not for bandwidth)."""
        total = self._exchange(full).reshape(-1)
        n = out.numel()
        out.copy_(total[self.rank * n:(self.rank + 1) * n].reshape(out.shape))
        return out

    def all_gather(self, own, full):
        import torch
        wide = torch.zeros(full.shape, dtype=full.dtype)
        n = own.numel()
        wide.reshape(-1)[self.rank * n:(self.rank + 1) * n] = own.detach().reshape(-1).cpu()
        full.copy_(self._exchange(wide).reshape(full.shape))
        return full

    def broadcast(self, t, root: int = 0):
        import torch
        src = t if self.rank == root else torch.zeros_like(t)
        t.copy_(self._exchange(src).reshape(t.shape))
        return t

    def reduce(self, t, root: int = 0):
        total = self._exchange(t)
        if self.rank == root:
            t.copy_(total.reshape(t.shape))
        return t

    def check(self) -> None:
        g = self.nm.groups.get(self.name)
        if g.state == "ERROR":
            raise ServiceError("GROUP_DESYNC", f"peer group {self.name!r}: {g.error}")

    def close(self) -> None:
        pass


class NetworkManager:
    def __init__(self, name: str, listen: str | None, store, state, chunk_bytes: int = P.CHUNK, device: int | None = None):
        self.name, self.listen_addr, self.store, self.state = name, listen, store, state
        self.device = device                 # CUDA ordinal of this daemon (None: CPU / virtual backend)
        self.handles: dict[str, Any] = {}    # group name -> what tasks see as ctx.groups[name]
        self.links: dict[str, Link] = {}
        self.lock = threading.RLock()
        self.groups = GroupTable()
        self.coll: dict[str, CollectiveQueue] = {}
        self.coll_inbox: dict[tuple[str, int], dict[str, Any]] = {}
        self.coll_cv = threading.Condition()
        self.core = PeerCore(name, self._emit, reserve=self._reserve, land=self._land, commit=self._commit, drop=self._drop,
                             chunk_bytes=chunk_bytes)
        self._stop = threading.Event()
        self._threads: list[threading.Thread] = []
        self._listener: socket.socket | None = None
        self.port: int | None = None

    # ------------------------------------------------------------------ store hooks of the core
    def _reserve(self, xid: str, size: int) -> None:
        self.store.reserve_inbound(xid, size)

    def _land(self, xid: str, off: int, payload) -> None:
        if payload is not None and len(payload):
            self.store.inbound_view(xid)[off:off + len(payload)] = payload

    def _commit(self, xid: str, dest: str | None):
        if dest is None:
            return self.store.inbound_view(xid)
        self.store.adopt_inbound(xid, dest)
        self.state.emit("peer_object_received", object=dest)
        return b""

    def _drop(self, xid: str) -> None:
        self.store.drop_inbound(xid)

    def _emit(self, peer: str, frame: dict, payload) -> None:
        link = self.links.get(peer)
        if link is None or not link.up:
            raise ServiceError("PEER_UNREACHABLE", f"no link to peer {peer!r}")
        link.send(frame, payload)

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> None:
        if self.listen_addr:
            host, _, port = self.listen_addr.rpartition(":")
            self._listener = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            self._listener.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            self._listener.bind((host or "127.0.0.1", int(port)))
            self._listener.listen(16)
            self._listener.settimeout(0.2)
            self.port = self._listener.getsockname()[1]
            self._spawn(self._accept_loop, "nm-accept")
        self._spawn(self._housekeeping_loop, "nm-housekeeping")

    def stop(self) -> None:
        self._stop.set()
        with self.lock:
            for l in list(self.links.values()):
                try:
                    l.send({"kind": "BYE"})
                except Exception:       # noqa: BLE001
                    pass
                l.up = False
                l.conn.close()
        if self._listener is not None:
            self._listener.close()
        for t in self._threads:
            t.join(timeout=2)

    def _spawn(self, fn, name, *args) -> None:
        t = threading.Thread(target=fn, args=args, name=name, daemon=True)
        t.start()
        self._threads.append(t)

    # ------------------------------------------------------------------ links
    def connect(self, peer: str, addr: str, timeout: float = 10.0) -> dict:
        host, _, port = addr.rpartition(":")
        try:
            s = socket.create_connection((host or "127.0.0.1", int(port)), timeout=timeout)
        except OSError as e:
            raise ServiceError("PEER_UNREACHABLE", f"cannot reach {peer!r} at {addr}: {e}") from None
        s.settimeout(None)
        s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        conn = Conn(s)
        conn.send({"kind": "HELLO", "name": self.name})
        hello, _ = conn.recv()
        if not hello or hello.get("kind") != "HELLO":
            conn.close()
            raise ServiceError("PEER_UNREACHABLE", f"{addr} did not answer the peer handshake")
        if hello["name"] != peer:
            conn.close()
            raise ServiceError("BAD_REQUEST", f"{addr} is peer {hello['name']!r}, not {peer!r}")
        self._adopt_link(peer, conn, outbound=True)
        return {"peer": peer, "addr": addr}

    def _adopt_link(self, peer: str, conn: Conn, outbound: bool) -> None:
        """Glare: if both sides dialled at once, the link opened by the smaller name survives."""
        with self.lock:
            old = self.links.get(peer)
            if old is not None and old.up:
                keep_outbound = self.name < peer
                if outbound != keep_outbound:
                    conn.close()
                    return
                old.up = False
                old.conn.close()
            link = Link(peer, conn, outbound)
            self.links[peer] = link
        self.state.emit("peer_link_up", peer=peer)
        self._spawn(self._reader_loop, f"nm-link-{peer}", link)

    def disconnect(self, peer: str) -> None:
        with self.lock:
            link = self.links.pop(peer, None)
        if link is not None:
            try:
                link.send({"kind": "BYE"})
            except Exception:       # noqa: BLE001
                pass
            self._link_down(link, "disconnected")

    def debug_sever(self, peer: str) -> None:
        """Cut the link without saying goodbye (host-side fault injection)."""
        link = self.links.get(peer)
        if link is not None:
            link.conn.close()

    def _link_down(self, link: Link, why: str) -> None:
        if not link.up:
            return
        link.up = False
        link.conn.close()
        with self.lock:
            self.core.peer_lost(link.peer)
        for g in self.groups.list():
            if link.peer in g["members"] and g["state"] != "ERROR":
                self.groups.mark_error(g["name"], f"link to {link.peer} went down ({why})")
                self._fan_out_group_error(g["name"], f"member {link.peer} unreachable")
        with self.coll_cv:
            self.coll_cv.notify_all()
        self.state.emit("peer_link_down", peer=link.peer, why=why)

    def _accept_loop(self) -> None:
        while not self._stop.is_set():
            try:
                s, _ = self._listener.accept()
            except socket.timeout:
                continue
            except OSError:
                return
            s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            conn = Conn(s)
            try:
                hello, _ = conn.recv()
                if not hello or hello.get("kind") != "HELLO":
                    conn.close()
                    continue
                conn.send({"kind": "HELLO", "name": self.name})
                self._adopt_link(hello["name"], conn, outbound=False)
            except (OSError, ValueError, ConnectionError):
                conn.close()

    def _reader_loop(self, link: Link) -> None:
        try:
            while link.up and not self._stop.is_set():
                frame, payload = link.conn.recv()
                if frame is None:
                    break
                link.last_heard = time.monotonic()
                link.bytes_in += 0 if payload is None else len(payload)
                kind = frame.get("kind")
                if kind == "PING":
                    link.send({"kind": "PONG"})
                elif kind == "PONG":
                    pass
                elif kind == "BYE":
                    break
                elif kind == "GROUP_JOIN":
                    self._on_group_join(link, frame)
                elif kind == "GROUP_ACK":
                    self.groups.ack(frame["group"], link.peer)
                elif kind == "GROUP_ERROR":
                    self.groups.mark_error(frame["group"], frame.get("why", "peer reported an error"))
                    with self.coll_cv:
                        self.coll_cv.notify_all()
                elif kind == "COLL":
                    with self.coll_cv:
                        self.coll_inbox.setdefault((frame["group"], int(frame["seq"])), {})[frame["from"]] = (frame, payload)
                        self.coll_cv.notify_all()
                else:
                    with self.lock:
                        self.core.handle(link.peer, frame, payload)
        except (OSError, ValueError, ConnectionError):
            pass
        finally:
            self._link_down(link, "connection closed")

    def _housekeeping_loop(self) -> None:
        while not self._stop.wait(P.HEARTBEAT_S / 4):
            now = time.monotonic()
            for link in list(self.links.values()):
                if not link.up:
                    continue
                if now - link.last_heard > P.LINK_DOWN_S:
                    self._link_down(link, "heartbeat lost")
                    continue
                try:
                    link.send({"kind": "PING"})
                except OSError:
                    self._link_down(link, "send failed")
            with self.lock:
                self.core.tick()

    # ------------------------------------------------------------------ object sends
    def send_object(self, peer: str, object_id: str, dest_id: str | None = None) -> str:
        if peer not in self.links or not self.links[peer].up:
            raise ServiceError("PEER_UNREACHABLE", f"no link to peer {peer!r}")
        view = self.store.view(object_id)
        with self.lock:
            return self.core.start_send(peer, object_id, view, dest_id)

    def transfer_status(self, xid: str) -> dict:
        with self.lock:
            return self.core.status(xid)

    def wait_transfer(self, xid: str, timeout: float = 60.0) -> dict:
        deadline = time.monotonic() + timeout
        while time.monotonic() < deadline:
            st = self.transfer_status(xid)
            if st["state"] in ("COMPLETE", "FAILED", "UNKNOWN"):
                return st
            time.sleep(0.002)
        return self.transfer_status(xid)

    def bw_probe(self, peer: str, mib: int = 64) -> dict:
        oid = f"__bwprobe_{self.name}"
        n = mib << 20
        self.store.create(oid, n, transient=True, replace=True)
        t0 = time.perf_counter()
        st = self.wait_transfer(self.send_object(peer, oid, oid + "_rx"), 120.0)
        dt = time.perf_counter() - t0
        self.store.release(oid, force=True)
        return {"peer": peer, "bytes": n, "seconds": dt, "gbs": n / dt / 1e9 if st["state"] == "COMPLETE" else 0.0, "state": st["state"]}

    # ------------------------------------------------------------------ groups
    def resolve_backend(self, backend: str, fake: bool) -> str:
        if backend != "auto":
            return backend
        return "hostmem" if fake else "nccl"

    def create_group(self, name: str, members: list[str], backend: str = "hostmem", timeout: float = 30.0, extra: dict | None = None) -> dict:
        if self.name not in members or members[0] != self.name:
            raise ServiceError("BAD_REQUEST", f"create_peer_group runs on the coordinator (first member); this daemon is {self.name!r}")
        missing = [m for m in members[1:] if m not in self.links or not self.links[m].up]
        if missing:
            raise ServiceError("PEER_UNREACHABLE", f"no link to group members {missing}")
        try:
            self.groups.create(name, members, backend, self.name)
        except KeyError:
            raise ServiceError("GROUP_EXISTS", f"peer group {name!r} already exists") from None
        self.coll[name] = CollectiveQueue(name)
        extra = dict(extra or {})
        if backend == "nccl":
            from .ncclcomm import NcclComm
            extra["nccl_uid"] = NcclComm.new_unique_id().hex()      # the unique id rides the join frame
        for m in members[1:]:
            self.links[m].send({"kind": "GROUP_JOIN", "group": name, "members": members, "backend": backend, "extra": extra})
        if len(members) == 1:
            self.groups.get(name).state = "READY"
        # the attachment barrier: every member builds its side of the backend before it acknowledges, this one meanwhile
        try:
            self._attach_backend(name, members, backend, extra)
        except Exception as e:      # noqa: BLE001
            self.groups.mark_error(name, f"backend {backend!r} did not attach on {self.name}: {e}")
            self._fan_out_group_error(name, self.groups.get(name).error)
            raise ServiceError("GROUP_DESYNC", self.groups.get(name).error) from None
        try:
            g = self.groups.wait_ready(name, timeout)
        except RuntimeError as e:
            raise ServiceError("GROUP_DESYNC", str(e)) from None
        return {"group": name, "members": list(g.members), "backend": backend, "rank": 0}

    def _attach_backend(self, name: str, members: list[str], backend: str, extra: dict) -> None:
        """This daemon's side of a group's collective backend; the result is what tasks get as ``ctx.groups[name]``."""
        rank = list(members).index(self.name)
        if backend == "nccl":
            from .ncclcomm import NcclComm
            if self.device is None:
                raise ServiceError("BAD_REQUEST", "the nccl lane needs a daemon on a CUDA device (CPU daemons use hostmem)")
            comm = NcclComm(name, rank, len(members), bytes.fromhex(extra["nccl_uid"]), int(self.device))
            comm.lane = "collective"
            comm.warm_up()
            self.handles[name] = comm
        else:
            self.handles[name] = HostGroupHandle(self, name)
        self.groups.get(name).comm = self.handles[name]

    def group_handles(self) -> dict:
        """Ready groups by name, as tasks see them (``TaskSpec.comm_groups`` names a group; ``ctx.groups[name]``)."""
        return {k: v for k, v in self.handles.items() if k in self.groups.groups and self.groups.get(k).state == "READY"}

    def _on_group_join(self, link: Link, frame: dict) -> None:
        name = frame["group"]
        self.groups.adopt(name, frame["members"], frame["backend"], link.peer)
        self.coll[name] = CollectiveQueue(name)
        try:
            self._attach_backend(name, list(frame["members"]), frame["backend"], dict(frame.get("extra") or {}))
        except Exception as e:      # noqa: BLE001
            self.groups.mark_error(name, f"backend {frame['backend']!r} did not attach on {self.name}: {e}")
            link.send({"kind": "GROUP_ERROR", "group": name, "why": self.groups.get(name).error})
            return
        link.send({"kind": "GROUP_ACK", "group": name})
        self.state.emit("peer_group_joined", group=name)

    def destroy_group(self, name: str) -> None:
        h = self.handles.pop(name, None)
        if h is not None and hasattr(h, "close"):
            try:
                h.close()
            except Exception:       # noqa: BLE001
                pass
        self.groups.drop(name)
        self.coll.pop(name, None)

    def _fan_out_group_error(self, name: str, why: str) -> None:
        try:
            g = self.groups.get(name)
        except KeyError:
            return
        for m in g.members:
            link = self.links.get(m)
            if m != self.name and link is not None and link.up:
                try:
                    link.send({"kind": "GROUP_ERROR", "group": name, "why": why})
                except OSError:
                    pass

    # ------------------------------------------------------------------ hostmem collectives (star, rank-ordered fp32)
    def all_reduce(self, group: str, array: np.ndarray, timeout: float = 60.0) -> np.ndarray:
        """Sum over the group, identical on every member (the coordinator adds in rank order)."""
        g = self.groups.get(group)
        if g.state != "READY":
            raise ServiceError("GROUP_DESYNC", f"peer group {group!r} is {g.state}: {g.error}")
        item = self.coll[group].push("all_reduce", array.nbytes, str(array.dtype))
        seq = item["seq"]
        hdr = {"kind": "COLL", "group": group, "seq": seq, "op": "all_reduce", "nbytes": array.nbytes, "dtype": str(array.dtype),
               "from": self.name}
        me = g.rank_of(self.name)
        if me != 0:
            self.links[g.coordinator].send(hdr, memoryview(np.ascontiguousarray(array)).cast("B"))
            frame, payload = self._await_coll(group, seq, [g.coordinator], timeout)[g.coordinator]
            self.coll[group].pending.popleft()
            return np.frombuffer(payload, dtype=array.dtype).reshape(array.shape).copy()
        got = self._await_coll(group, seq, list(g.members[1:]), timeout)
        acc = array.astype(np.float32, copy=True)
        for m in g.members[1:]:
            frame, payload = got[m]
            if (frame["op"], int(frame["nbytes"]), frame["dtype"]) != ("all_reduce", array.nbytes, str(array.dtype)):
                self.groups.mark_error(group, f"collective #{seq}: member {m} issued {frame['op']} of {frame['nbytes']} bytes")
                self._fan_out_group_error(group, self.groups.get(group).error)
                raise ServiceError("GROUP_DESYNC", self.groups.get(group).error)
            acc += np.frombuffer(payload, dtype=array.dtype).reshape(array.shape).astype(np.float32)
        out = acc.astype(array.dtype)
        for m in g.members[1:]:
            self.links[m].send(hdr, memoryview(out).cast("B"))
        self.coll[group].pending.popleft()
        return out

    def _await_coll(self, group: str, seq: int, senders: list[str], timeout: float) -> dict:
        deadline = time.monotonic() + timeout
        with self.coll_cv:
            while True:
                box = self.coll_inbox.get((group, seq), {})
                if all(s in box for s in senders):
                    return self.coll_inbox.pop((group, seq))
                g = self.groups.get(group)
                if g.state == "ERROR":
                    raise ServiceError("GROUP_DESYNC", f"peer group {group!r}: {g.error}")
                left = deadline - time.monotonic()
                if left <= 0:
                    self.groups.mark_error(group, f"collective #{seq} timed out waiting for {[s for s in senders if s not in box]}")
                    raise ServiceError("GROUP_DESYNC", self.groups.get(group).error)
                self.coll_cv.wait(min(left, 0.1))

    # ------------------------------------------------------------------ introspection
    def list_peers(self) -> list[dict]:
        now = time.monotonic()
        return [{"peer": l.peer, "up": l.up, "outbound": l.outbound, "silent_s": round(now - l.last_heard, 3),
                 "bytes_out": l.bytes_out, "bytes_in": l.bytes_in} for l in self.links.values()]
