"""Which source (rank) is responsible for which byte range of which logical object: the input of the
checkpoint source policy and of restore plans.  Replicated objects list every rank for the whole span; ZeRO
slices list one rank per slice; tensor / expert shards list the owner of each packed region.
Role parity: reference ``src/dataflow_training/distributed/responsibility.py:46``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping

from .parallelism import ParallelismScheme
from .sharding import zero_slices


@dataclass(frozen=True)
class Span:
    source: int
    lo: int
    hi: int
    replica: bool = False


def responsibility_map(objects: Mapping[str, int], scheme: ParallelismScheme,
                       kinds: Mapping[str, str] | None = None) -> dict[str, list[Span]]:
    """``objects``: logical id -> bytes.  ``kinds[id]`` in {"parameter", "optimizer_state", "other"} (default:
    by prefix W_/O_).  Under dp/zero3 parameters and optimizer state are sliced; under zero1* only optimizer
    state; under ``co`` and solo everything is replicated on (or private to) every rank."""
    world = scheme.world
    dp = scheme.axis("dp")
    resp = (dp.responsibility or "zero3") if dp else None
    out: dict[str, list[Span]] = {}
    for oid, nbytes in objects.items():
        kind = (kinds or {}).get(oid) or ("parameter" if oid.startswith("W_") else "optimizer_state" if oid.startswith("O_") else "other")
        sliced = dp is not None and dp.size > 1 and (
            (resp == "zero3" and kind in ("parameter", "optimizer_state")) or
            (resp in ("zero1", "zero1rs") and kind == "optimizer_state"))
        if sliced:
            spans = []
            for r in range(world):
                k = scheme.coords(r)[dp.name]
                lo, ln = zero_slices(nbytes, dp.size)[k]
                if ln:
                    # ranks that differ only on other axes hold replicas of the same slice
                    first = min(x for x in range(world) if scheme.coords(x)[dp.name] == k)
                    spans.append(Span(r, lo, lo + ln, replica=r != first))
            out[oid] = spans
        else:
            out[oid] = [Span(r, 0, int(nbytes), replica=r != 0) for r in range(world)]
    return out
