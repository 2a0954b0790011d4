"""In-process and child-process daemons for tests and tools (role of the reference's
``testing/server_process.py`` and ``run/driver.engine_client``)."""
from __future__ import annotations

import contextlib
import os
import tempfile
import threading
import time

from ..service import EngineClient, EngineConfig, Server


@contextlib.contextmanager
def engine_client(backing_gib: float = 0.25, *, device=None, fake: bool = False, socket_path: str | None = None,
                  kernel_set: str | None = None, peer_name: str | None = None, peer_listen: str | None = None,
                  poison_on_free: bool = False):
    """Boot a daemon in a thread of this process and yield a connected client."""
    from ..register import register_all
    register_all()
    path = socket_path or os.path.join(tempfile.mkdtemp(prefix="dfd-"), "d.sock")
    server = Server(EngineConfig(socket_path=path, slab_backing_gib=backing_gib, device=device, fake=fake,
                                 kernel_set=kernel_set, peer_name=peer_name, peer_listen=peer_listen,
                                 poison_on_free=poison_on_free))
    t = threading.Thread(target=server.serve_forever, name=f"engine-server:{path}", daemon=True)
    t.start()
    client = None
    for _ in range(3000):
        try:
            client = EngineClient(path, client_name="in-process")
            break
        except (ConnectionError, FileNotFoundError, OSError):
            if not t.is_alive():
                raise RuntimeError("daemon thread died during boot")
            time.sleep(0.01)
    if client is None:
        raise RuntimeError("daemon did not accept connections")
    client.server = server
    try:
        yield client
    finally:
        client.close()
        server.state.shutdown_requested.set()
        t.join(timeout=30)


# ------------------------------------------------------------------------------------------------ daemons in processes of their own
_LAUNCH = """
import sys
from dataflow_b200.service import EngineConfig, Server
from dataflow_b200.register import register_all
register_all()
{extra}
Server(EngineConfig(socket_path=sys.argv[1], slab_backing_gib=float(sys.argv[2]),
                    device=None if sys.argv[3] == "cpu" else int(sys.argv[3]), fake=sys.argv[4] == "1",
                    poison_on_free=sys.argv[5] == "1", kernel_set=sys.argv[6] or None)).serve_forever()
"""


class ServerProcess:
    """A daemon running in a child process, with a client connected to it.  ``close()`` asks it to shut down, then makes
    sure the process is gone (terminate, then kill, by pid: never by name)."""

    def __init__(self, proc, socket_path: str, client: EngineClient, log_path: str):
        self.proc, self.socket_path, self.client, self.log_path = proc, socket_path, client, log_path

    @property
    def alive(self) -> bool:
        return self.proc.poll() is None

    def log_tail(self, n: int = 40) -> str:
        try:
            with open(self.log_path, encoding="utf-8", errors="replace") as f:
                return "".join(f.readlines()[-n:])
        except OSError:
            return ""

    def close(self) -> None:
        try:
            if self.alive:
                try:
                    self.client.shutdown()
                except (OSError, ConnectionError, RuntimeError):
                    pass
            self.client.close()
        except Exception:      # noqa: BLE001  (a dead daemon's socket may fail in any way; the process is reaped below)
            pass
        for sig_wait in (10.0, 5.0):
            try:
                self.proc.wait(timeout=sig_wait)
                break
            except Exception:  # noqa: BLE001  (subprocess.TimeoutExpired)
                (self.proc.terminate if sig_wait == 10.0 else self.proc.kill)()
        if self.proc.poll() is None:
            self.proc.kill()
            self.proc.wait(timeout=10)


def spawn_server(backing_gib: float = 0.25, *, device=None, fake: bool = False, poison_on_free: bool = False,
                 kernel_set: str | None = None, extra_source: str = "", socket_path: str | None = None,
                 boot_timeout: float = 120.0, env: dict | None = None) -> ServerProcess:
    """Start a daemon in a fresh interpreter and connect to it.  ``extra_source`` runs in the child after the built-in
    resolver kinds are registered and before it serves (a test registers a resolver of its own that way)."""
    import subprocess
    import sys
    work = tempfile.mkdtemp(prefix="dfd-proc-")
    path = socket_path or os.path.join(work, "d.sock")
    log_path = os.path.join(work, "daemon.log")
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    child_env = dict(os.environ)
    child_env["PYTHONPATH"] = root + os.pathsep + child_env.get("PYTHONPATH", "")
    child_env.update(env or {})
    with open(log_path, "wb") as log:
        proc = subprocess.Popen([sys.executable, "-c", _LAUNCH.format(extra=extra_source), path, str(backing_gib),
                                 "cpu" if device is None else str(int(device)), "1" if fake else "0", "1" if poison_on_free else "0",
                                 kernel_set or ""], stdout=log, stderr=subprocess.STDOUT, env=child_env, start_new_session=True)
    deadline = time.monotonic() + boot_timeout
    client = None
    while time.monotonic() < deadline:
        if proc.poll() is not None:
            with open(log_path, encoding="utf-8", errors="replace") as f:
                raise RuntimeError(f"the daemon exited with {proc.returncode} while booting:\n{f.read()[-2000:]}")
        try:
            client = EngineClient(path, client_name="test-client")
            break
        except (ConnectionError, FileNotFoundError, OSError):
            time.sleep(0.05)
    if client is None:
        proc.kill()
        proc.wait(timeout=10)
        raise RuntimeError(f"the daemon did not accept connections within {boot_timeout} s")
    return ServerProcess(proc, path, client, log_path)


@contextlib.contextmanager
def out_of_process_server(backing_gib: float = 0.25, **kw):
    """A daemon of its own for one ``with`` block (a test that needs its own boot options); yields the client, with the
    process handle on ``client.server_process``."""
    sp = spawn_server(backing_gib, **kw)
    sp.client.server_process = sp
    try:
        yield sp.client
    finally:
        sp.close()


class SharedServer:
    """One daemon for a whole test run.  ``fresh()`` returns a client on a blank daemon: programs unregistered, objects
    wiped (protected ones too).  If a test left the daemon dead, or in a state the wipe cannot clear, it is replaced by a
    new one (``respawns`` counts how often), so one broken test does not fail the ones after it."""

    def __init__(self, backing_gib: float = 0.25, **spawn_kw):
        self.backing_gib, self.spawn_kw = backing_gib, spawn_kw
        self.sp: ServerProcess | None = None
        self.respawns = 0

    def _blank(self) -> bool:
        sp = self.sp
        if sp is None or not sp.alive:
            return False
        try:
            for p in sp.client.list_programs():
                sp.client.unregister_program(p["prog_id"] if isinstance(p, dict) else p)
            sp.client.wipe(scope="all", force=True)
            return not sp.client.list_objects() and sp.client.health().get("ok", True)
        except (OSError, ConnectionError, RuntimeError, KeyError):
            return False

    def fresh(self) -> EngineClient:
        if not self._blank():
            if self.sp is not None:
                self.sp.close()
                self.respawns += 1
            self.sp = spawn_server(self.backing_gib, **self.spawn_kw)
        return self.sp.client

    def close(self) -> None:
        if self.sp is not None:
            self.sp.close()
            self.sp = None
