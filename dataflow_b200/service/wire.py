"""Wire protocol of the engine service: one JSON line per message, optionally followed by
``payload_bytes`` raw bytes.  Schema tag, error codes and the program content id are the
reference's (``src/dataflow/service/wire.py:22-164``) so clients interoperate."""
from __future__ import annotations

import json
import socket
from typing import Any

from ..core.jsonio import program_content_id  # noqa: F401  (re-exported: clients gate on computed == registered id)

SCHEMA_VERSION = "dataflow-service/s1"

ERROR_CODES = (
    "SCHEMA_VERSION_SKEW", "BAD_REQUEST", "UNKNOWN_OP", "UNKNOWN_OBJECT", "UNKNOWN_PROGRAM", "UNKNOWN_RUN",
    "UNKNOWN_SNAPSHOT", "UNKNOWN_RESTORE", "BINDING_MISMATCH", "MISSING_INPUTS", "CAPACITY", "PROTECTED", "LEASED",
    "RUN_FAILED", "CANCELLED", "IO_ERROR", "VERSION_SKEW", "COLLISION", "VERIFY_FAILED", "GROUP_EXISTS",
    "GROUP_DESYNC", "PEER_UNREACHABLE", "PEER_DISABLED", "INTERNAL",
)


class ServiceError(Exception):
    def __init__(self, code: str, message: str = "", **detail: Any):
        if code not in ERROR_CODES:
            code = "INTERNAL"
        super().__init__(f"{code}: {message}")
        self.code, self.message, self.detail = code, message, detail

    def to_dict(self) -> dict[str, Any]:
        return {"ok": False, "error": {"code": self.code, "message": self.message, **self.detail}}


class Conn:
    """Framed connection: ``send(obj, payload)`` / ``recv() -> (obj, payload)``."""

    def __init__(self, sock: socket.socket):
        self.sock = sock
        self.rfile = sock.makefile("rb", buffering=1 << 20)

    def send(self, obj: dict[str, Any], payload: bytes | memoryview | None = None) -> None:
        if payload is not None:
            obj = dict(obj, payload_bytes=len(payload))
        self.sock.sendall(json.dumps(obj, separators=(",", ":")).encode() + b"\n")
        if payload is not None and len(payload):
            self.sock.sendall(payload)

    def recv(self, into: memoryview | None = None) -> tuple[dict[str, Any] | None, bytes | memoryview | None]:
        line = self.rfile.readline()
        if not line:
            return None, None
        obj = json.loads(line)
        n = int(obj.get("payload_bytes", 0) or 0)
        payload = None
        if n:
            if into is not None and len(into) >= n:
                got, view = 0, into[:n]
                while got < n:
                    k = self.rfile.readinto(view[got:])
                    if not k:
                        raise ConnectionError("peer closed mid-payload")
                    got += k
                payload = view
            else:
                payload = self.rfile.read(n)
                if len(payload) != n:
                    raise ConnectionError("peer closed mid-payload")
        return obj, payload

    def close(self) -> None:
        try:
            self.rfile.close()
            self.sock.close()
        except OSError:
            pass
