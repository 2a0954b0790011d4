"""Test transport for the peer plane: an in-memory link between two ``PeerCore``s with a scripted ``FaultPlan``
(drop / duplicate / corrupt the n-th frame of a kind).  Faults are made on the host, in the message path — never on
a device.  Parity: reference ``src/dataflow/service/peer/transports.py:19-80``.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field


@dataclass
class FaultPlan:
    """``drop={"CHUNK": {1}}`` drops the 2nd CHUNK frame (0-based) that crosses the link, and so on."""
    drop: dict[str, set[int]] = field(default_factory=dict)
    duplicate: dict[str, set[int]] = field(default_factory=dict)
    corrupt: dict[str, set[int]] = field(default_factory=dict)
    seen: dict[str, int] = field(default_factory=dict)
    log: list[tuple[str, str]] = field(default_factory=list)

    def apply(self, frame: dict, payload):
        """Returns the list of (frame, payload) that actually cross the link."""
        kind = frame["kind"]
        i = self.seen.get(kind, 0)
        self.seen[kind] = i + 1
        if i in self.drop.get(kind, ()):
            self.log.append(("drop", f"{kind}#{i}"))
            return []
        if i in self.corrupt.get(kind, ()) and payload is not None and len(payload):
            b = bytearray(payload)
            b[len(b) // 2] ^= 0x5A
            payload = bytes(b)
            self.log.append(("corrupt", f"{kind}#{i}"))
        out = [(frame, payload)]
        if i in self.duplicate.get(kind, ()):
            out.append((dict(frame), payload))
            self.log.append(("duplicate", f"{kind}#{i}"))
        return out


class MemLink:
    """Two endpoints ``a`` and ``b``; ``pump()`` delivers queued frames until the link is quiet."""

    def __init__(self, plan_ab: FaultPlan | None = None, plan_ba: FaultPlan | None = None):
        self.q: deque = deque()
        self.plans = {"ab": plan_ab or FaultPlan(), "ba": plan_ba or FaultPlan()}
        self.cores: dict[str, object] = {}

    def attach(self, side: str, core) -> None:
        self.cores[side] = core

    def emitter(self, side: str):
        other, plan = ("b", self.plans["ab"]) if side == "a" else ("a", self.plans["ba"])

        def emit(peer, frame, payload):
            data = None if payload is None else bytes(payload)
            for fr, pl in plan.apply(frame, data):
                self.q.append((other, side, fr, pl))
        return emit

    def pump(self, limit: int = 100000) -> int:
        n = 0
        while self.q and n < limit:
            to, frm, frame, payload = self.q.popleft()
            self.cores[to].handle(self.cores[frm].name, frame, payload)
            n += 1
        return n
