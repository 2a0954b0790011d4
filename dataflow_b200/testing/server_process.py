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
