"""Catalog of named resident objects over one host slab (pinned when a CUDA backend owns it).

First-fit offset allocator (4 KiB alignment), put / get / release / protect / wipe / duplicate,
inbound reservations for the peer plane, scratch, and **read leases**: a snapshot leases the objects
it copies; a run that would mutate a leased object is parked until the lease is released.
Role parity: reference ``src/dataflow/service/store.py:26-460`` and ``hostmem.py:25-92``.
"""
from __future__ import annotations

import ctypes
import threading
from dataclasses import dataclass, field

from ..runtime import SlabAllocator
from .wire import ServiceError

ALIGN = 4096
SYSTEM_RESERVE_GIB = 12


def auto_cap_bytes() -> int:
    """Slab size for ``slab_backing_gib="auto"``: host RAM minus a system reserve."""
    try:
        import os
        total = os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES")
    except (ValueError, OSError):
        total = 32 << 30
    return max(total - (SYSTEM_RESERVE_GIB << 30), 1 << 30)


class HostSlab:
    """One contiguous host region; ``backend`` (a CudaBackend) pins it, else plain memory."""

    def __init__(self, nbytes: int, backend=None):
        self.nbytes = int(nbytes)
        self.backend = backend
        self._buf = None
        if backend is not None and hasattr(backend, "pin_region"):
            self.base = backend.pin_region(self.nbytes, False)
        else:
            self._buf = (ctypes.c_char * self.nbytes)()
            self.base = ctypes.addressof(self._buf)

    def bytes_view(self, offset: int, size: int) -> memoryview:
        return memoryview((ctypes.c_char * size).from_address(self.base + offset)).cast("B")

    def close(self) -> None:
        if self.backend is not None and self._buf is None and self.base:
            self.backend.unpin_region(self.base, self.nbytes)
        self.base, self._buf = 0, None


@dataclass
class Resident:
    id: str
    offset: int
    size: int
    protected: bool = False
    leases: int = 0
    transient: bool = False
    meta: dict = field(default_factory=dict)


class Store:
    def __init__(self, slab: HostSlab):
        self.slab = slab
        self.alloc = SlabAllocator(slab.nbytes, ALIGN)
        self.objects: dict[str, Resident] = {}
        self.inbound: dict[str, Resident] = {}
        self.lock = threading.RLock()
        self.created_log: list[str] | None = None

    # -- allocation
    def _carve(self, size: int) -> int:
        off = self.alloc.allocate(max(int(size), 1))
        if off is None:
            raise ServiceError("CAPACITY", f"backing slab cannot hold {size} more bytes "
                                           f"(used {self.alloc.used()} of {self.alloc.capacity()})")
        return off

    def create(self, oid: str, size: int, *, transient: bool = False, replace: bool = False) -> Resident:
        with self.lock:
            if oid in self.objects:
                cur = self.objects[oid]
                if not replace:
                    raise ServiceError("COLLISION", f"object {oid!r} already exists")
                if cur.size == size and not cur.leases:
                    return cur
                self.release(oid, force=True)
            r = Resident(oid, self._carve(size), int(size), transient=transient)
            self.objects[oid] = r
            if self.created_log is not None:
                self.created_log.append(oid)
            return r

    def put(self, oid: str, data: bytes | memoryview, *, replace: bool = True) -> Resident:
        r = self.create(oid, len(data), replace=replace)
        if r.leases:
            raise ServiceError("LEASED", f"object {oid!r} is leased by a snapshot")
        self.view(oid)[:len(data)] = data
        return r

    def get(self, oid: str) -> Resident:
        try:
            return self.objects[oid]
        except KeyError:
            raise ServiceError("UNKNOWN_OBJECT", f"no object {oid!r}") from None

    def view(self, oid: str) -> memoryview:
        r = self.get(oid)
        return self.slab.bytes_view(r.offset, r.size)

    def address(self, oid: str) -> int:
        return self.slab.base + self.get(oid).offset

    def release(self, oid: str, force: bool = False) -> None:
        with self.lock:
            r = self.get(oid)
            if r.protected and not force:
                raise ServiceError("PROTECTED", f"object {oid!r} is protected")
            if r.leases:
                raise ServiceError("LEASED", f"object {oid!r} is leased")
            self.alloc.release(r.offset)
            del self.objects[oid]

    def protect(self, oid: str, on: bool = True) -> None:
        self.get(oid).protected = on

    def duplicate(self, src: str, dst: str) -> Resident:
        with self.lock:
            s = self.get(src)
            d = self.create(dst, s.size, replace=True)
            self.view(dst)[:] = self.view(src)
            return d

    def wipe(self, scope: str = "unprotected", force: bool = False) -> int:
        with self.lock:
            n = 0
            for oid in list(self.objects):
                r = self.objects[oid]
                if r.leases:
                    if force:
                        continue
                    raise ServiceError("LEASED", f"object {oid!r} is leased")
                if r.protected and not (scope == "all" and force):
                    continue
                self.alloc.release(r.offset)
                del self.objects[oid]
                n += 1
            return n

    # -- leases
    def acquire_leases(self, ids) -> None:
        with self.lock:
            for oid in ids:
                self.get(oid)
            for oid in ids:
                self.objects[oid].leases += 1

    def release_leases(self, ids) -> None:
        with self.lock:
            for oid in ids:
                r = self.objects.get(oid)
                if r is not None and r.leases:
                    r.leases -= 1

    def leased(self, ids) -> list[str]:
        return [i for i in ids if i in self.objects and self.objects[i].leases]

    # -- peer plane: land inbound bytes in a reserved extent, adopt under the final name when complete
    def reserve_inbound(self, key: str, size: int) -> Resident:
        with self.lock:
            r = Resident(key, self._carve(size), int(size))
            self.inbound[key] = r
            return r

    def inbound_view(self, key: str) -> memoryview:
        r = self.inbound[key]
        return self.slab.bytes_view(r.offset, r.size)

    def adopt_inbound(self, key: str, oid: str) -> Resident:
        with self.lock:
            r = self.inbound.pop(key)
            if oid in self.objects:
                self.release(oid, force=True)
            r.id = oid
            self.objects[oid] = r
            return r

    def drop_inbound(self, key: str) -> None:
        with self.lock:
            r = self.inbound.pop(key, None)
            if r is not None:
                self.alloc.release(r.offset)

    # -- failed-run rollback
    def begin_created_log(self) -> None:
        self.created_log = []

    def rollback_created(self) -> None:
        for oid in self.created_log or ():
            if oid in self.objects and not self.objects[oid].leases:
                self.release(oid, force=True)
        self.created_log = None

    def end_created_log(self) -> None:
        self.created_log = None

    def query(self) -> dict:
        return {"capacity": self.alloc.capacity(), "used": self.alloc.used(), "peak": self.alloc.peak(),
                "objects": len(self.objects), "largest_free": self.alloc.largest_free()}
