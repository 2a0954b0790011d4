"""Peer groups: named member lists with an attachment barrier.  The coordinator (first member) creates a group by
sending GROUP_JOIN down each link; a member attaches its backend and answers GROUP_ACK; the group is ready when
every member has acknowledged.  Parity: reference ``src/dataflow/service/peer/groups.py:23-114``.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field


@dataclass
class GroupRecord:
    name: str
    members: tuple[str, ...]
    backend: str
    coordinator: str
    acked: set = field(default_factory=set)
    state: str = "FORMING"             # FORMING -> READY | ERROR
    error: str = ""
    comm: object = None

    def rank_of(self, member: str) -> int:
        return self.members.index(member)


class GroupTable:
    def __init__(self):
        self.lock = threading.Condition()
        self.groups: dict[str, GroupRecord] = {}

    def create(self, name: str, members, backend: str, coordinator: str) -> GroupRecord:
        with self.lock:
            if name in self.groups and self.groups[name].state != "ERROR":
                raise KeyError(f"peer group {name!r} already exists")
            g = GroupRecord(name, tuple(members), backend, coordinator)
            self.groups[name] = g
            return g

    def adopt(self, name: str, members, backend: str, coordinator: str) -> GroupRecord:
        """Member side of GROUP_JOIN."""
        with self.lock:
            g = GroupRecord(name, tuple(members), backend, coordinator, state="READY")
            self.groups[name] = g
            return g

    def ack(self, name: str, member: str) -> None:
        with self.lock:
            g = self.groups.get(name)
            if g is None:
                return
            g.acked.add(member)
            if g.acked >= set(g.members) - {g.coordinator}:
                g.state = "READY"
            self.lock.notify_all()

    def wait_ready(self, name: str, timeout: float = 30.0) -> GroupRecord:
        with self.lock:
            ok = self.lock.wait_for(lambda: self.groups[name].state in ("READY", "ERROR"), timeout)
            g = self.groups[name]
            if not ok:
                g.state, g.error = "ERROR", f"members {sorted(set(g.members) - g.acked - {g.coordinator})} never acknowledged"
            if g.state == "ERROR":
                raise RuntimeError(f"peer group {name!r}: {g.error}")
            return g

    def mark_error(self, name: str, why: str) -> None:
        with self.lock:
            g = self.groups.get(name)
            if g is not None:
                g.state, g.error = "ERROR", why
                self.lock.notify_all()

    def drop(self, name: str) -> None:
        with self.lock:
            self.groups.pop(name, None)

    def get(self, name: str) -> GroupRecord:
        with self.lock:
            return self.groups[name]

    def list(self) -> list[dict]:
        with self.lock:
            return [{"name": g.name, "members": list(g.members), "backend": g.backend, "state": g.state, "error": g.error}
                    for g in self.groups.values()]
