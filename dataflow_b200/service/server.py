"""dataflowd: the engine behind a unix-socket service with a persistent object store.

Three planes share one process: *control* (JSON verbs), *data* (raw payloads that land directly
in store extents) and *peer* (links to other daemons, ``service.peer``).  Threads: the accept loop,
one thread per client connection, ONE dispatcher thread that owns the store mutations and the engine
(FIFO; a ``run`` that would touch leased objects is parked and retried when leases drop), a payload
thread per snapshot / restore job.  Role parity: reference ``src/dataflow/service/server.py:49-554``.
"""
from __future__ import annotations

import os
import queue
import socket
import threading
import time
import traceback
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Callable

from .store import HostSlab, Store, auto_cap_bytes
from .wire import SCHEMA_VERSION, Conn, ServiceError


@dataclass
class EngineConfig:
    socket_path: str = "/tmp/dataflowd.sock"
    slab_backing_gib: float | str = 1.0            # GiB or "auto"
    device: int | None = 0                         # CUDA ordinal; None = host backend
    kernel_set: str | None = None
    fake: bool = False                             # virtual-time backend (no device work)
    poison_on_free: bool = False
    peer_name: str | None = None
    peer_listen: str | None = None                 # "host:port"
    peer_chunk_bytes: int = 128 << 20
    peer_rdma_device: str | None = None
    peer_coll_scratch_mib: int = 512
    peer_bw_probe_mib: int = 128
    host_bw_probe_mib: int = 256


class EngineState:
    """Ids, counters and the event ring."""

    def __init__(self, ring: int = 4096):
        self.lock = threading.Lock()
        self.next_run = 0
        self.next_job = 0
        self.events: deque[dict] = deque(maxlen=ring)
        self.event_seq = 0
        self.counters: dict[str, int] = {}
        self.started = time.time()
        self.shutdown_requested = threading.Event()

    def new_id(self, prefix: str) -> str:
        with self.lock:
            if prefix == "r":
                self.next_run += 1
                return f"r-{self.next_run:06d}"
            self.next_job += 1
            return f"{prefix}-{self.next_job:06d}"

    def emit(self, kind: str, **fields: Any) -> None:
        with self.lock:
            self.event_seq += 1
            self.events.append({"seq": self.event_seq, "t": time.time(), "kind": kind, **fields})
            self.counters[kind] = self.counters.get(kind, 0) + 1

    def events_since(self, seq: int) -> list[dict]:
        with self.lock:
            return [e for e in self.events if e["seq"] > seq]


@dataclass
class _Call:
    fn: Callable[[], Any]
    done: threading.Event = field(default_factory=threading.Event)
    result: Any = None
    error: BaseException | None = None
    parked_until: float = 0.0


class Dispatcher(threading.Thread):
    """Single FIFO worker that owns store mutations and the engine."""

    def __init__(self, state: EngineState):
        super().__init__(name="dataflowd-dispatcher", daemon=True)
        self.q: "queue.Queue[_Call | None]" = queue.Queue()
        self.parked: list[_Call] = []
        self.state = state

    def submit(self, fn: Callable[[], Any]) -> Any:
        c = _Call(fn)
        self.q.put(c)
        c.done.wait()
        if c.error is not None:
            raise c.error
        return c.result

    def unpark_all(self) -> None:
        for c in self.parked:
            self.q.put(c)
        self.parked = []

    def run(self) -> None:
        while True:
            try:
                c = self.q.get(timeout=0.05)
            except queue.Empty:
                if self.parked:
                    self.unpark_all()
                continue
            if c is None:
                return
            try:
                c.result = c.fn()
            except ServiceError as e:
                if e.code == "LEASED" and e.detail.get("park"):
                    self.parked.append(c)            # retried when leases are released
                    continue
                c.error = e
            except BaseException as e:               # noqa: BLE001
                c.error = ServiceError("INTERNAL", f"{type(e).__name__}: {e}", traceback=traceback.format_exc()[-2000:])
            c.done.set()

    def stop(self) -> None:
        self.q.put(None)


FAST_VERBS = {"health", "engine_status", "session_status", "run_status", "list_runs", "run_events", "list_programs",
              "list_resolvers", "query_object", "list_objects", "query_backing", "query_fast", "snapshot_status",
              "restore_status", "list_peers", "peer_status", "transfer_status", "list_peer_groups", "subscribe_events"}
CRITICAL_VERBS = {"cancel_run", "shutdown"}


class Server:
    def __init__(self, config: EngineConfig):
        self.config = config
        self.state = EngineState()
        self.dispatcher = Dispatcher(self.state)
        self.store: Store | None = None
        self.slab: HostSlab | None = None
        self.backend = None
        self.handlers: dict[str, Callable[[dict, bytes | None], Any]] = {}
        self.programs: dict[str, dict] = {}
        self.runs: dict[str, dict] = {}
        self.jobs: dict[str, dict] = {}
        self.cancel_events: dict[str, threading.Event] = {}
        self.nm = None
        self._sock: socket.socket | None = None
        self._threads: list[threading.Thread] = []

    # -- boot
    def boot(self) -> None:
        from ..runtime import CpuBackend, FakeBackend
        cfg = self.config
        if cfg.fake:
            self.backend = FakeBackend()
        elif cfg.device is not None and _cuda_ok():
            from ..runtime import CudaBackend
            import torch
            torch.cuda.set_device(cfg.device)
            self.backend = CudaBackend(cfg.device, "poll")
        else:
            self.backend = CpuBackend()
            self.config.device = None
        nbytes = auto_cap_bytes() if cfg.slab_backing_gib == "auto" else int(float(cfg.slab_backing_gib) * (1 << 30))
        pin = self.backend if (not cfg.fake and self.config.device is not None) else None
        self.slab = HostSlab(nbytes, pin)
        self.store = Store(self.slab)
        self.host_bw = {}
        if not cfg.fake and cfg.host_bw_probe_mib:
            from .hostbw import measure_host_bw
            try:
                self.host_bw = measure_host_bw(self.slab, cfg.host_bw_probe_mib, self.config.device)
            except Exception as e:       # noqa: BLE001  (a probe never keeps a daemon from booting)
                self.host_bw = {"error": f"{type(e).__name__}: {e}"}
        from . import handlers, snapshots
        handlers.install(self)
        snapshots.install(self)
        if cfg.peer_name:
            from .peer.nm import NetworkManager
            from . import handlers_peers
            self.nm = NetworkManager(cfg.peer_name, cfg.peer_listen, self.store, self.state,
                                     chunk_bytes=cfg.peer_chunk_bytes, device=None if cfg.fake else cfg.device)
            self.nm.start()
            handlers_peers.install(self)

    # -- serving
    def serve_forever(self) -> None:
        path = self.config.socket_path
        if os.path.exists(path):
            probe = socket.socket(socket.AF_UNIX)
            try:
                probe.connect(path)
                probe.close()
                raise RuntimeError(f"a daemon is already serving {path}")
            except (ConnectionRefusedError, FileNotFoundError):
                os.unlink(path)                      # stale socket: reclaim
            finally:
                probe.close()
        self.boot()
        self.dispatcher.start()
        self._sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self._sock.bind(path)
        self._sock.listen(64)
        self._sock.settimeout(0.2)
        self.state.emit("daemon_up", socket=path)
        try:
            while not self.state.shutdown_requested.is_set():
                try:
                    c, _ = self._sock.accept()
                except socket.timeout:
                    continue
                except OSError:
                    break
                t = threading.Thread(target=self._serve_conn, args=(c,), name="dataflowd-conn", daemon=True)
                t.start()
                self._threads.append(t)
        finally:
            self.teardown()

    def teardown(self) -> None:
        # order: stop accepting -> peers -> dispatcher -> engine/backend -> slab -> socket file
        try:
            if self._sock is not None:
                self._sock.close()
        except OSError:
            pass
        if self.nm is not None:
            self.nm.stop()
        self.dispatcher.stop()
        self.dispatcher.join(timeout=10)
        from . import handlers
        handlers.close_engine(self)
        if self.slab is not None:
            self.slab.close()
        try:
            os.unlink(self.config.socket_path)
        except OSError:
            pass

    def _serve_conn(self, sock: socket.socket) -> None:
        conn = Conn(sock)
        try:
            hello, _ = conn.recv()
            if hello is None:
                return
            if hello.get("schema") != SCHEMA_VERSION:
                conn.send(ServiceError("SCHEMA_VERSION_SKEW", f"server speaks {SCHEMA_VERSION}, client sent "
                                                              f"{hello.get('schema')!r}").to_dict())
                return
            conn.send({"ok": True, "schema": SCHEMA_VERSION, "server": "dataflow_b200", "pid": os.getpid()})
            while True:
                req, payload = conn.recv()
                if req is None:
                    return
                out_payload = None
                try:
                    res = self._route(req, payload)
                    if isinstance(res, tuple):
                        res, out_payload = res
                    reply = {"ok": True, **(res or {})}
                except ServiceError as e:
                    reply = e.to_dict()
                except Exception as e:           # noqa: BLE001
                    reply = ServiceError("INTERNAL", f"{type(e).__name__}: {e}").to_dict()
                conn.send(reply, out_payload)
                if req.get("op") == "shutdown":
                    return
        except (ConnectionError, OSError, ValueError):
            pass
        finally:
            conn.close()

    def _route(self, req: dict, payload):
        op = req.get("op")
        h = self.handlers.get(op)
        if h is None:
            raise ServiceError("UNKNOWN_OP", f"unknown verb {op!r}")
        if op in FAST_VERBS or op in CRITICAL_VERBS:
            return h(req, payload)
        return self.dispatcher.submit(lambda: h(req, payload))


def _cuda_ok() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False
