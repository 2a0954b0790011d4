"""Transport-free rendezvous state machines of the peer plane.

``PeerCore`` owns every in-flight send and receive of one daemon.  It never touches a socket: the owner feeds it
frames (``handle``) and time (``tick``), and it answers through two callbacks — ``emit(peer, frame, payload)`` to
put a frame on the wire and the store hooks ``reserve / land / commit / drop`` to place bytes.  That makes the
protocol testable against scripted loss, duplication and corruption without any network
(``tests/test_peer_plane.py``).  Contract parity: reference ``src/dataflow/service/peer/core.py:85-424``.
"""
from __future__ import annotations

import itertools
from collections import OrderedDict, deque
from dataclasses import dataclass, field
from typing import Any, Callable

from . import protocol as P


@dataclass
class SenderMachine:
    xid: str
    peer: str
    object_id: str
    dest_id: str
    data: memoryview
    crc: int
    state: str = "RTS_SENT"            # RTS_SENT -> STREAMING -> DONE_SENT -> COMPLETE | FAILED
    retries: int = 0
    next_retry: float = 0.0
    last_progress: float = 0.0
    resends: int = 0
    error: str = ""


@dataclass
class ReceiverMachine:
    xid: str
    peer: str
    dest_id: str
    size: int
    crc: int
    received: int = 0
    seen: set = field(default_factory=set)        # chunk offsets already landed (duplicates are ignored)
    state: str = "RECEIVING"                      # RECEIVING -> COMMITTED | FAILED
    last_progress: float = 0.0


class PeerCore:
    def __init__(self, name: str, emit: Callable[[str, dict, bytes | memoryview | None], None], *,
                 reserve: Callable[[str, int], None], land: Callable[[str, int, Any], None],
                 commit: Callable[[str, str], bytes | memoryview], drop: Callable[[str], None],
                 chunk_bytes: int = P.CHUNK, clock: Callable[[], float] | None = None):
        import time
        self.name, self.emit = name, emit
        self.reserve, self.land, self.commit, self.drop = reserve, land, commit, drop
        self.chunk_bytes = chunk_bytes
        self.clock = clock or time.monotonic
        self.senders: dict[str, SenderMachine] = {}
        self.receivers: dict[str, ReceiverMachine] = {}
        self.finished: "OrderedDict[str, dict]" = OrderedDict()        # xid -> the DONE_ACK we answered with
        self._seq = itertools.count(1)
        self.stats = {"sent": 0, "received": 0, "nacks": 0, "resends": 0, "duplicates": 0, "failed": 0}

    # ------------------------------------------------------------------ sending
    def start_send(self, peer: str, object_id: str, data, dest_id: str | None = None) -> str:
        xid = f"{self.name}-{next(self._seq)}"
        mv = memoryview(data).cast("B")
        m = SenderMachine(xid, peer, object_id, dest_id or object_id, mv, P.checksum(mv), last_progress=self.clock())
        self.senders[xid] = m
        self._send_rts(m)
        return xid

    def _send_rts(self, m: SenderMachine) -> None:
        eager = len(m.data) <= P.EAGER_MAX
        self.emit(m.peer, P.rts(m.xid, m.object_id, len(m.data), m.crc, m.dest_id, inline=b"" if eager else None),
                  m.data if eager else None)
        m.state = "DONE_SENT" if eager else "RTS_SENT"

    def _stream(self, m: SenderMachine) -> None:
        m.state = "STREAMING"
        for off in range(0, max(len(m.data), 1), self.chunk_bytes):
            part = m.data[off:off + self.chunk_bytes]
            self.emit(m.peer, P.chunk(m.xid, off, len(part)), part)
        self.emit(m.peer, P.done(m.xid), None)
        m.state = "DONE_SENT"
        m.last_progress = self.clock()

    # ------------------------------------------------------------------ frames in
    def handle(self, peer: str, frame: dict, payload=None) -> None:
        kind = frame.get("kind")
        fn = getattr(self, "_on_" + str(kind).lower(), None)
        if fn is not None:
            fn(peer, frame, payload)

    def _on_rts(self, peer, f, payload):
        xid = f["xid"]
        if xid in self.finished:                         # duplicate of a transfer we already committed
            self.stats["duplicates"] += 1
            self.emit(peer, self.finished[xid], None)
            return
        if xid in self.receivers:
            self.stats["duplicates"] += 1
            if not f.get("eager"):
                self.emit(peer, P.cts(xid), None)
            return
        try:
            self.reserve(xid, int(f["size"]))
        except Exception as e:                           # noqa: BLE001  no room (or a name clash): the sender retries
            self.stats["nacks"] += 1
            self.emit(peer, P.nack(xid, f"{type(e).__name__}: {e}"), None)
            return
        r = ReceiverMachine(xid, peer, f["dest"], int(f["size"]), int(f["crc"]), last_progress=self.clock())
        self.receivers[xid] = r
        if f.get("eager"):
            self.land(xid, 0, payload if payload is not None else b"")
            r.received = r.size
            self._finish_receive(r)
        else:
            self.emit(peer, P.cts(xid), None)

    def _on_cts(self, peer, f, payload):
        m = self.senders.get(f["xid"])
        if m is not None and m.state == "RTS_SENT":
            self._stream(m)

    def _on_nack(self, peer, f, payload):
        m = self.senders.get(f["xid"])
        if m is None or m.state not in ("RTS_SENT", "DONE_SENT"):
            return
        m.retries += 1
        if m.retries > P.NACK_RETRIES:
            self._fail_send(m, f"receiver refused {m.retries} times: {f.get('reason')}")
            return
        m.state = "BACKOFF"
        m.next_retry = self.clock() + P.NACK_BACKOFF_S * (2 ** (m.retries - 1))

    def _on_chunk(self, peer, f, payload):
        r = self.receivers.get(f["xid"])
        if r is None or r.state != "RECEIVING":
            return
        off = int(f["offset"])
        if off in r.seen:
            self.stats["duplicates"] += 1
            return
        self.land(r.xid, off, payload)
        r.seen.add(off)
        r.received += int(f["size"])
        r.last_progress = self.clock()

    def _on_done(self, peer, f, payload):
        xid = f["xid"]
        if xid in self.finished:
            self.stats["duplicates"] += 1
            self.emit(peer, self.finished[xid], None)
            return
        r = self.receivers.get(xid)
        if r is None:
            return
        if r.received < r.size:
            # chunks were lost: ask for the whole payload again (chunks are offset-addressed: re-landing is harmless)
            r.seen.clear()
            r.received = 0
            self.emit(peer, P.done_ack(xid, False, "incomplete"), None)
            return
        self._finish_receive(r)

    def _finish_receive(self, r: ReceiverMachine) -> None:
        data = self.commit(r.xid, None)                  # peek: bytes of the reservation
        if P.checksum(data) != r.crc:
            r.seen.clear()
            r.received = 0
            self.emit(r.peer, P.done_ack(r.xid, False, "checksum"), None)
            return
        self.commit(r.xid, r.dest_id)
        r.state = "COMMITTED"
        ack = P.done_ack(r.xid, True)
        self.finished[r.xid] = ack
        while len(self.finished) > P.DEDUP_RING:
            self.finished.popitem(last=False)
        del self.receivers[r.xid]
        self.stats["received"] += 1
        self.emit(r.peer, ack, None)

    def _on_done_ack(self, peer, f, payload):
        m = self.senders.get(f["xid"])
        if m is None or m.state == "COMPLETE":
            return
        if f.get("ok"):
            m.state = "COMPLETE"
            self.stats["sent"] += 1
            return
        m.resends += 1
        self.stats["resends"] += 1
        if m.resends > P.NACK_RETRIES:
            self._fail_send(m, f"receiver rejected the payload {m.resends} times ({f.get('reason')})")
            return
        if len(m.data) <= P.EAGER_MAX:
            self._send_rts(m)
        else:
            self._stream(m)

    # ------------------------------------------------------------------ time
    def tick(self, now: float | None = None) -> None:
        now = self.clock() if now is None else now
        for m in list(self.senders.values()):
            if m.state == "BACKOFF" and now >= m.next_retry:
                self._send_rts(m)
                m.last_progress = now
            elif m.state in ("RTS_SENT", "DONE_SENT", "STREAMING") and now - m.last_progress > P.INACTIVITY_S:
                self._fail_send(m, "no progress (inactivity timeout)")
        for r in list(self.receivers.values()):
            if now - r.last_progress > P.INACTIVITY_S:
                r.state = "FAILED"
                self.drop(r.xid)
                del self.receivers[r.xid]
                self.stats["failed"] += 1

    def _fail_send(self, m: SenderMachine, why: str) -> None:
        m.state, m.error = "FAILED", why
        self.stats["failed"] += 1

    def peer_lost(self, peer: str) -> None:
        for m in self.senders.values():
            if m.peer == peer and m.state not in ("COMPLETE", "FAILED"):
                self._fail_send(m, f"link to {peer} went down")
        for r in list(self.receivers.values()):
            if r.peer == peer:
                self.drop(r.xid)
                del self.receivers[r.xid]

    def status(self, xid: str) -> dict:
        m = self.senders.get(xid)
        if m is None:
            return {"xid": xid, "state": "UNKNOWN"}
        return {"xid": xid, "state": m.state, "peer": m.peer, "object": m.object_id, "bytes": len(m.data), "retries": m.retries,
                "resends": m.resends, "error": m.error}


class CollectiveQueue:
    """Per-group FIFO of collective requests: members must issue the same sequence; a mismatch is an error, not a hang."""

    def __init__(self, group: str):
        self.group = group
        self.pending: deque[dict] = deque()
        self.seq = 0

    def push(self, op: str, nbytes: int, dtype: str) -> dict:
        self.seq += 1
        item = {"seq": self.seq, "op": op, "nbytes": int(nbytes), "dtype": dtype}
        self.pending.append(item)
        return item

    def match(self, remote: dict) -> dict:
        if not self.pending:
            raise RuntimeError(f"group {self.group}: peer issued {remote['op']} #{remote['seq']} but nothing is pending here")
        mine = self.pending[0]
        if (mine["seq"], mine["op"], mine["nbytes"], mine["dtype"]) != (remote["seq"], remote["op"], remote["nbytes"], remote["dtype"]):
            raise RuntimeError(f"group {self.group}: collective mismatch: local {mine} vs remote {remote}")
        return self.pending.popleft()
