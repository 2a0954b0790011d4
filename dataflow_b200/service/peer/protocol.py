"""Peer plane frames and constants.

An object send is a rendezvous: ``RTS`` (sender announces id, size, checksum; small objects ride inline — the
eager path) -> ``CTS`` (receiver reserved room) or ``NACK`` (no room yet: the sender backs off and retries) ->
``CHUNK`` x n (offset-addressed, so duplicates and re-sends are idempotent) -> ``DONE`` (sender finished) ->
``DONE_ACK`` (receiver verified the crc32 and committed, or asks for a resend).  Every frame carries the transfer
id ``xid``; receivers remember finished ``xid``s in a ring so a duplicated ``RTS`` or ``DONE`` is answered, not
re-executed.  Contract parity: reference ``src/dataflow/service/peer/protocol.py:36-91``.
"""
from __future__ import annotations

import zlib
from typing import Any

EAGER_MAX = 64 << 10               # objects up to this size ride inside the RTS frame
CHUNK = 128 << 20                  # payload bytes per CHUNK frame
NACK_BACKOFF_S = 0.1               # first retry delay; doubles each time
NACK_RETRIES = 5
INACTIVITY_S = 60.0                # a transfer with no progress for this long fails
DEDUP_RING = 256
HEARTBEAT_S = 2.0
LINK_DOWN_S = 6.0

KINDS = ("HELLO", "PING", "PONG", "RTS", "CTS", "NACK", "CHUNK", "DONE", "DONE_ACK", "GROUP_JOIN", "GROUP_ACK",
         "GROUP_ERROR", "COLL", "BYE")


def checksum(data) -> int:
    return zlib.crc32(data) & 0xFFFFFFFF


def rts(xid: str, object_id: str, size: int, crc: int, dest_id: str | None = None, inline: bytes | None = None) -> dict[str, Any]:
    return {"kind": "RTS", "xid": xid, "id": object_id, "dest": dest_id or object_id, "size": int(size), "crc": int(crc),
            "eager": inline is not None}


def cts(xid: str) -> dict[str, Any]:
    return {"kind": "CTS", "xid": xid}


def nack(xid: str, reason: str) -> dict[str, Any]:
    return {"kind": "NACK", "xid": xid, "reason": reason}


def chunk(xid: str, offset: int, size: int) -> dict[str, Any]:
    return {"kind": "CHUNK", "xid": xid, "offset": int(offset), "size": int(size)}


def done(xid: str) -> dict[str, Any]:
    return {"kind": "DONE", "xid": xid}


def done_ack(xid: str, ok: bool, reason: str = "") -> dict[str, Any]:
    return {"kind": "DONE_ACK", "xid": xid, "ok": bool(ok), "reason": reason}
