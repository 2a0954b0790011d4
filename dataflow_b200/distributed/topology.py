"""Where ranks run: hosts, devices, groups.  A topology is a TOML file

    [hosts.box]            # address = "user@host" (omit for the local machine), backing_gib, repo
    devices = [0, 1, 2, 3]
    [groups.train]
    members = ["box:0", "box:1", "box:2", "box:3"]      # rank = position; the first member coordinates

or is made on the fly for this machine (``local_topology``).
Role parity: reference ``src/dataflow_training/distributed/topology.py:27-210``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class HostSpec:
    name: str
    address: str | None = None               # None: this machine; else an ssh destination
    devices: tuple[int, ...] = (0,)
    backing_gib: float | str = "auto"
    repo: str | None = None                  # checkout path on that host
    python: str = "python"

    @property
    def local(self) -> bool:
        return self.address in (None, "", "localhost", "127.0.0.1")


@dataclass(frozen=True)
class Member:
    host: str
    device: int

    @property
    def key(self) -> str:
        return f"{self.host}:{self.device}"


@dataclass(frozen=True)
class GroupSpec:
    name: str
    members: tuple[Member, ...]
    backend: str = "auto"

    @property
    def world(self) -> int:
        return len(self.members)

    @property
    def coordinator(self) -> Member:
        return self.members[0]


@dataclass
class Topology:
    hosts: dict[str, HostSpec] = field(default_factory=dict)
    groups: dict[str, GroupSpec] = field(default_factory=dict)

    def group(self, name: str | None = None) -> GroupSpec:
        if name is None:
            if len(self.groups) != 1:
                raise KeyError(f"topology has groups {sorted(self.groups)}: name one")
            return next(iter(self.groups.values()))
        return self.groups[name]

    def host_of(self, m: Member) -> HostSpec:
        return self.hosts[m.host]

    def validate(self) -> "Topology":
        for g in self.groups.values():
            seen = set()
            for m in g.members:
                if m.host not in self.hosts:
                    raise ValueError(f"group {g.name!r}: unknown host {m.host!r}")
                if m.device not in self.hosts[m.host].devices:
                    raise ValueError(f"group {g.name!r}: host {m.host!r} has no device {m.device}")
                if m.key in seen:
                    raise ValueError(f"group {g.name!r}: member {m.key} listed twice")
                seen.add(m.key)
        return self

    def socket_path(self, m: Member, root: str = "/tmp") -> str:
        return f"{root}/dataflowd.{m.host}.{m.device}.sock"


def _parse(d: Mapping[str, Any]) -> Topology:
    hosts = {}
    for name, h in (d.get("hosts") or {}).items():
        hosts[name] = HostSpec(name, h.get("address"), tuple(h.get("devices", [0])),
                               h.get("backing_gib", h.get("slab_gib", "auto")), h.get("repo"), h.get("python", "python"))
    groups = {}
    for name, g in (d.get("groups") or {}).items():
        members = []
        for m in g["members"]:
            host, _, dev = str(m).partition(":")
            members.append(Member(host, int(dev or 0)))
        groups[name] = GroupSpec(name, tuple(members), g.get("backend", "auto"))
    return Topology(hosts, groups).validate()


def load_topology(path: str) -> Topology:
    import tomllib
    with open(path, "rb") as f:
        return _parse(tomllib.load(f))


def local_topology(n_devices: int = 1, backing_gib: float | str = "auto", group: str = "local") -> Topology:
    host = HostSpec("local", None, tuple(range(n_devices)), backing_gib)
    return Topology({"local": host}, {group: GroupSpec(group, tuple(Member("local", i) for i in range(n_devices)))}).validate()


def local_pair_topology(backing_gib: float | str = "auto") -> Topology:
    return local_topology(2, backing_gib, "pair")
