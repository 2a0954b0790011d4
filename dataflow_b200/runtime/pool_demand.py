"""What a program asks of the session pools, found by running it on the virtual-time backend before the real pools exist.

The plan says how many bytes are live at the worst moment; the pools have to serve those bytes through an allocator, and
two things the plan's ledger does not see decide whether they can:

    the backing pool    holds every backing copy that is NOT one of the caller's own buffers (the host store holds the
                        persistent objects for the whole run, whether or not a backing copy "exists" in the plan's eyes at a
                        given moment), so its demand is not the plan's backing peak minus the store's size: it is the peak
                        of the transient copies alone, which only a run shows;
    the fast pool       is an offset allocator over one region: at a fill of 98 % a request can fail for want of a
                        contiguous hole although enough bytes are free.

``dry_run_pools`` executes the program for a few steps on ``FakeBackend`` (no memory is touched, no kernel runs; tasks and
transfers take their planned times) with the fast pool at its real size and an unbounded backing pool, and reports per
pool the peak in use and the requests the slab could not serve.  The trainer sizes the backing pool from it and, when
the fast pool overflows, plans again with a little less memory while keeping the pool as large as it was.
Reference role: the pool prewarm from a dry run's ``pool_demand`` (``src/dataflow/runtime/pool.py:276-318``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping

from ..core import Program


@dataclass(frozen=True)
class PoolDemand:
    fast_capacity: int
    fast_peak: int
    fast_overflows: int               # in the last (steady) step
    fast_overflow_bytes: int          # bytes the slab could not serve in that step
    backing_peak: int                 # of what the session's backing pool holds: transient copies only
    backing_overflows: int
    steps: int

    @property
    def fits(self) -> bool:
        return self.fast_overflows == 0 and self.backing_overflows == 0


def dry_run_pools(program: Program, caller_buffers: Mapping[str, int], fast_capacity: int, *, backing_capacity: int | None = None,
                  keep_resident: bool = False, dispatch_ahead: int = 0, fast_tail: int = 0, steps: int = 2) -> PoolDemand:
    """``caller_buffers``: id -> bytes of the objects the caller hands to ``execute`` itself (the host store).
    ``backing_capacity``: None = unbounded (measure the demand); a number = check a pool of that size."""
    from . import Engine, FakeBackend, Session
    from .executable import Buffer
    be = FakeBackend()
    ses = Session(be)
    total = sum(int(v) + 4096 for v in caller_buffers.values()) + 4096
    base = be.alloc(1, total)
    bufs, off = {}, 0
    for oid, n in caller_buffers.items():
        bufs[oid] = Buffer(base + off, int(n), "backing", oid)
        off += (int(n) + 4095) // 4096 * 4096
    if fast_tail:
        ses.native.set_fast_tail(int(fast_tail))
    unbounded = max(4 * int(program_backing_bytes(program)), 64 << 30)
    ses.native.ensure_pools(int(fast_capacity), int(backing_capacity) if backing_capacity is not None else unbounded, 0.0, False)
    eng = Engine(be, session=ses)
    f_prev = b_prev = 0
    f_last = b_last = 0
    log_from = 0
    for s in range(max(steps, 1)):
        res = eng.execute(program, None, bufs, run_args={"step": s + 1}, manage_pools=False, keep_resident=keep_resident,
                          dispatch_ahead=dispatch_ahead)
        res.raise_if_failed()
        fs, bs = ses.native.fast_pool_stats(), ses.native.backing_pool_stats()
        f_last, b_last = fs["overflows"] - f_prev, bs["overflows"] - b_prev
        log_from = f_prev
        f_prev, b_prev = fs["overflows"], bs["overflows"]
    asked = [a for a, _, _ in fs["overflow_log"][log_from:log_from + f_last]]
    missing = f_last - len(asked)                        # the log keeps the first 64: price the rest at the largest seen
    over_bytes = sum(asked) + (max(asked) * missing if asked and missing > 0 else 0)
    out = PoolDemand(int(fs["capacity"]), int(fs["peak"]), int(f_last), int(over_bytes), int(bs["peak"]), int(b_last), steps)
    ses.native.drop_resident()
    be.free(1, base, total)
    return out


def program_backing_bytes(program: Program) -> int:
    """An upper bound of what can ever sit in backing memory: every object once."""
    return sum(program.object_sizes().values())
