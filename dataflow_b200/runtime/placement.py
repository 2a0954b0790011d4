"""Static placement: every fast-memory allocation of a step gets a slab offset computed ahead of time.

A dry run of the annotated program on the virtual-time backend records, in order, every fast allocation and release
(``Engine.execute(record_allocs=True)``).  From that log each allocation becomes an interval in *allocation-event order*
(the k-th allocation of an object until its release, or the end of the run); ``compute_placement`` packs the intervals
into offsets so that intervals that overlap in time never overlap in address — first fit over several deterministic
orders and seeded restarts, keeping the packing with the lowest top.  The engine then places every buffer at its
planned offset (``SlabAllocator::allocate_at``); if the realised order of events ever differs from the recorded one
and the bytes are still taken, that one allocation falls back to the dynamic allocator (counted in
``placement_escapes``) and the run goes on.  With a placement there is no fragmentation, no slab overflow, and buffers
keep their addresses from step to step.
Reference role: ``src/dataflow/runtime/placement.py:40-159`` (``PlacementRecorder``, ``compute_placement``,
``PlacementError``).
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field

ALIGN = 512


class PlacementError(RuntimeError):
    pass


@dataclass(frozen=True)
class Lifetime:
    object_id: str
    occurrence: int          # k-th fast allocation of the object in the run
    size: int                # bytes, rounded up to the slab alignment
    start: int               # position in the allocation log
    end: int                 # position of the release (exclusive), or the length of the log


@dataclass
class Placement:
    offsets: dict[tuple[str, int], int]
    top: int                                  # bytes of slab the packing needs
    lifetimes: list[Lifetime] = field(default_factory=list)

    def for_index(self, chain_index) -> list[list[int]]:
        """Per object index of the executor's program form: offsets of its 1st, 2nd, ... allocation (-1 = dynamic)."""
        out: list[list[int]] = [[] for _ in chain_index.ir_object_ids]
        for (oid, k), off in self.offsets.items():
            i = chain_index.index.get(oid)
            if i is None:
                continue
            lst = out[i]
            while len(lst) <= k:
                lst.append(-1)
            lst[k] = int(off)
        return out


def _round(n: int) -> int:
    return (max(int(n), 1) + ALIGN - 1) // ALIGN * ALIGN


def lifetimes_from_log(allocs, margin: int = 0) -> list[Lifetime]:
    """``allocs``: the (object id | None, size, pointer, kind) log of a run (kind 1 allocated, 2 held from the previous run,
    0 released).  ``margin`` widens every lifetime by that many log positions on both sides: on a device, copies finish at
    slightly different points of the chain than in the dry run, and a widened lifetime keeps its bytes clear of neighbours
    that arrive a little early or leave a little late."""
    open_by_ptr: dict[int, tuple[str, int, int, int]] = {}
    count: dict[str, int] = {}
    out: list[Lifetime] = []
    n = len(allocs)
    for pos, (oid, size, ptr, kind) in enumerate(allocs):
        if kind in (1, 2):
            k = count.get(oid, 0)
            count[oid] = k + 1
            open_by_ptr[ptr] = (oid, k, _round(size), 0 if kind == 2 else pos)
        else:
            rec = open_by_ptr.pop(ptr, None)
            if rec is not None:
                out.append(Lifetime(rec[0], rec[1], rec[2], max(rec[3] - margin, 0), min(pos + margin, n)))
    for oid, k, size, start in open_by_ptr.values():
        out.append(Lifetime(oid, k, size, max(start - margin, 0), n))
    out.sort(key=lambda lt: (lt.start, lt.object_id, lt.occurrence))
    return out


def record_lifetimes(program, margin: int = 0) -> list[Lifetime]:
    """Dry run on the virtual-time backend (synthetic executables occupy the compute lane for the planned durations)."""
    from . import Engine, FakeBackend, synthetic_resolver
    res = Engine(FakeBackend()).execute(program, synthetic_resolver, record_allocs=True)
    res.raise_if_failed()
    return lifetimes_from_log(res.stats["allocs"], margin)


def _first_fit(order: list[Lifetime], capacity: int | None) -> tuple[dict, int] | None:
    import numpy as np
    n = len(order)
    off = np.zeros(n, dtype=np.int64)
    size = np.zeros(n, dtype=np.int64)
    start = np.zeros(n, dtype=np.int64)
    end = np.zeros(n, dtype=np.int64)
    offsets: dict[tuple[str, int], int] = {}
    top = 0
    for i, lt in enumerate(order):
        live = (start[:i] < lt.end) & (end[:i] > lt.start)          # already placed and alive at some point of this lifetime
        at = 0
        if live.any():
            o, s = off[:i][live], size[:i][live]
            idx = np.argsort(o, kind="stable")
            for a, b in zip(o[idx].tolist(), s[idx].tolist()):
                if a - at >= lt.size:
                    break
                at = max(at, a + b)
        if capacity is not None and at + lt.size > capacity:
            return None
        off[i], size[i], start[i], end[i] = at, lt.size, lt.start, lt.end
        offsets[(lt.object_id, lt.occurrence)] = at
        top = max(top, at + lt.size)
    return offsets, top


def compute_placement(lifetimes: list[Lifetime], capacity: int | None = None, restarts: int = 8, seed: int = 0,
                      search_s: float = 6.0) -> Placement:
    """Pack ``lifetimes`` into ``capacity`` bytes (``None`` = unbounded).  Deterministic orders first (by size, by duration,
    by start, and run-long objects first then by start), then seeded perturbations, then — only when nothing fits yet — a
    local search that moves short runs of the best order around for at most ``search_s`` seconds.  Raises ``PlacementError``
    when no tried order fits."""
    import time
    n_log = max((lt.end for lt in lifetimes), default=0)
    orders = [sorted(lifetimes, key=lambda lt: (-lt.size, lt.start)),
              sorted(lifetimes, key=lambda lt: (-(lt.end - lt.start), -lt.size)),
              sorted(lifetimes, key=lambda lt: (lt.start, -lt.size)),
              sorted(lifetimes, key=lambda lt: (0 if (lt.end - lt.start) > n_log // 2 else 1, lt.start, -lt.size))]
    rng = random.Random(seed)
    for _ in range(restarts):
        o = list(orders[0])
        # perturb the size order locally: swaps between neighbours keep big blocks early
        for i in range(len(o) - 1):
            if rng.random() < 0.3:
                o[i], o[i + 1] = o[i + 1], o[i]
        orders.append(o)
    best = None
    for o in orders:
        got = _first_fit(o, capacity)
        if got is not None and (best is None or got[1] < best[1]):
            best = got
    if best is None and capacity is not None and lifetimes and search_s > 0:
        # unbounded tops tell which order is closest; walk from there
        scored = sorted(((_first_fit(o, None)[1], i) for i, o in enumerate(orders[:4])))
        cur, cur_top = list(orders[scored[0][1]]), scored[0][0]
        t_end = time.time() + search_s
        while time.time() < t_end and cur_top > capacity:
            o = list(cur)
            i, ln, j = rng.randrange(len(o)), rng.randint(1, 8), rng.randrange(len(o))
            blk = o[i:i + ln]
            del o[i:i + ln]
            o[j:j] = blk
            top = _first_fit(o, None)[1]
            if top <= cur_top:
                cur, cur_top = o, top
        if cur_top <= capacity:
            best = _first_fit(cur, capacity)
    if best is None:
        peak = peak_live_bytes(lifetimes)
        raise PlacementError(f"no packing of {len(lifetimes)} allocations fits {capacity} bytes (their peak live size is {peak})")
    return Placement(best[0], best[1], list(lifetimes))


def peak_live_bytes(lifetimes: list[Lifetime]) -> int:
    events = []
    for lt in lifetimes:
        events.append((lt.start, 1, lt.size))
        events.append((lt.end, 0, -lt.size))
    live = peak = 0
    for _, _, d in sorted(events):
        live += d
        peak = max(peak, live)
    return peak


def plan_placement(program, capacity: int | None = None, margin: int = 6, **kw) -> Placement:
    """Placement for a real device: lifetimes widened by ``margin`` log positions (exact lifetimes if that does not fit)."""
    try:
        return compute_placement(record_lifetimes(program, margin), capacity, **kw)
    except PlacementError:
        if not margin:
            raise
        return compute_placement(record_lifetimes(program, 0), capacity, **kw)
