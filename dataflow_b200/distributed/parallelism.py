"""Parallelism as data: named axes over a rank grid, compiled from CLI flags and stamped into programs.

An ``Axis`` is one way of splitting work (``dp`` rounds / ZeRO state, ``tp`` tensor + sequence parallel, ``ep``
experts, ``pp`` stages); a ``ParallelismScheme`` is an ordered list of axes whose sizes multiply to the world
size, rank-major in the LAST axis (the fastest-varying axis is the one that should sit on the closest links:
tp inside the NVSwitch domain).  Unlike the reference, whose ``validate`` refuses more than one axis
(``src/dataflow_training/distributed/parallelism.py:197-243``), meshes such as ``dp x tp`` and ``dp x ep`` are
first class here.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Sequence

AXIS_KINDS = ("dp", "tp", "ep", "pp")
DP_RESPONSIBILITIES = ("zero3", "zero1rs", "zero1", "co")


class SchemeError(ValueError):
    pass


@dataclass(frozen=True)
class Axis:
    name: str
    kind: str
    size: int
    responsibility: str | None = None            # dp: who owns which optimizer state
    rank_rounds: tuple[int, ...] | None = None   # dp: grad-accum rounds per rank (weighted data parallel)
    sequence_parallel: bool = False              # tp: norm / residual regions sharded on the sequence dim
    options: Mapping[str, Any] = field(default_factory=dict)

    def to_dict(self) -> dict:
        return {"name": self.name, "kind": self.kind, "size": self.size, "responsibility": self.responsibility,
                "rank_rounds": list(self.rank_rounds) if self.rank_rounds else None,
                "sequence_parallel": self.sequence_parallel, "options": dict(self.options)}


@dataclass(frozen=True)
class ParallelismScheme:
    axes: tuple[Axis, ...] = ()

    # -- constructors
    @staticmethod
    def solo() -> "ParallelismScheme":
        return ParallelismScheme(())

    @staticmethod
    def data_parallel(world: int | None = None, rank_rounds: Sequence[int] | None = None,
                      responsibility: str = "zero3") -> "ParallelismScheme":
        n = world if world is not None else len(rank_rounds or ())
        return ParallelismScheme((Axis("dp", "dp", int(n), responsibility, tuple(rank_rounds) if rank_rounds else None),))

    @staticmethod
    def tensor_parallel(size: int, sequence_parallel: bool = True, **options) -> "ParallelismScheme":
        return ParallelismScheme((Axis("tp", "tp", int(size), sequence_parallel=sequence_parallel, options=options),))

    @staticmethod
    def expert_parallel(size: int, **options) -> "ParallelismScheme":
        return ParallelismScheme((Axis("ep", "ep", int(size), options=options),))

    @staticmethod
    def mesh(*axes: Axis) -> "ParallelismScheme":
        return ParallelismScheme(tuple(axes))

    # -- facts
    @property
    def world(self) -> int:
        n = 1
        for a in self.axes:
            n *= a.size
        return n

    def axis(self, kind: str) -> Axis | None:
        return next((a for a in self.axes if a.kind == kind), None)

    def validate(self, world: int | None = None) -> "ParallelismScheme":
        seen = set()
        for a in self.axes:
            if a.kind not in AXIS_KINDS:
                raise SchemeError(f"axis {a.name!r}: unknown kind {a.kind!r} (one of {AXIS_KINDS})")
            if a.name in seen or any(b.kind == a.kind and b is not a for b in self.axes):
                raise SchemeError(f"axis kind {a.kind!r} appears twice")
            seen.add(a.name)
            if a.size < 1:
                raise SchemeError(f"axis {a.name!r}: size {a.size}")
            if a.kind == "dp":
                if (a.responsibility or "zero3") not in DP_RESPONSIBILITIES:
                    raise SchemeError(f"dp responsibility {a.responsibility!r} is not one of {DP_RESPONSIBILITIES}")
                if a.rank_rounds is not None and (len(a.rank_rounds) != a.size or min(a.rank_rounds) < 1):
                    raise SchemeError(f"dp rank_rounds {a.rank_rounds} must give every one of {a.size} ranks >= 1 round")
            elif a.responsibility or a.rank_rounds:
                raise SchemeError(f"axis {a.name!r}: responsibility / rank_rounds belong to a dp axis")
        kinds = [a.kind for a in self.axes]
        if "tp" in kinds and "ep" in kinds:
            raise SchemeError("tp and ep in one scheme: experts are sharded whole (ep) or by columns (tp), not both")
        if "tp" in kinds and kinds[-1] != "tp":
            raise SchemeError("the tp axis must be the last (fastest-varying) one: its collectives sit on the hot path")
        if world is not None and self.world != world:
            raise SchemeError(f"scheme covers {self.world} ranks, the job has {world}")
        return self

    def coords(self, rank: int) -> dict[str, int]:
        """Position of ``rank`` on every axis (row-major, last axis fastest)."""
        out, r = {}, int(rank)
        for a in reversed(self.axes):
            out[a.name] = r % a.size
            r //= a.size
        return {a.name: out[a.name] for a in self.axes}

    def group_members(self, axis_name: str, rank: int) -> list[int]:
        """Ranks that share every coordinate with ``rank`` except the one on ``axis_name``."""
        me = self.coords(rank)
        return [r for r in range(self.world) if all(v == me[k] for k, v in self.coords(r).items() if k != axis_name)]

    def rounds_of(self, rank: int, default_rounds: int) -> int:
        dp = self.axis("dp")
        if dp is None or dp.rank_rounds is None:
            return default_rounds
        return dp.rank_rounds[self.coords(rank)[dp.name]]

    def to_dict(self) -> dict:
        return {"axes": [a.to_dict() for a in self.axes], "world": self.world}

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "ParallelismScheme":
        axes = []
        for a in d.get("axes", ()):
            axes.append(Axis(a["name"], a["kind"], int(a["size"]), a.get("responsibility"),
                             tuple(a["rank_rounds"]) if a.get("rank_rounds") else None, bool(a.get("sequence_parallel")),
                             dict(a.get("options") or {})))
        return ParallelismScheme(tuple(axes))


def scheme_from_flags(world: int, *, opt_shard: str = "zero3", rounds: Sequence[int] | None = None, tp: int = 1,
                      ep: int = 1, sequence_parallel: bool = True) -> ParallelismScheme:
    """``--gpus / --opt-shard / --rounds / --tp / --ep`` -> scheme.  The remaining factor of the world is dp."""
    if world == 1:
        return ParallelismScheme.solo()
    inner = tp * ep
    if world % inner:
        raise SchemeError(f"tp={tp} x ep={ep} does not divide the world size {world}")
    dp = world // inner
    axes = []
    if dp > 1 or inner == 1:
        axes.append(Axis("dp", "dp", dp, opt_shard, tuple(rounds) if rounds else None))
    if ep > 1:
        axes.append(Axis("ep", "ep", ep))
    if tp > 1:
        axes.append(Axis("tp", "tp", tp, sequence_parallel=sequence_parallel))
    return ParallelismScheme(tuple(axes)).validate(world)
