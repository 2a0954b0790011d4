"""From responsibilities to what each checkpoint source writes.

``simple``: every source writes everything it holds (replicas included: the record then certifies them equal —
a drift tripwire, at world x the bytes).  ``dedup``: of a replicated span only the lowest-index holder writes.
Private per-source state (ids in ``private``) is always written by its holder under a source-qualified id.
Role parity: reference ``src/dataflow_training/distributed/source_policy.py:52-160``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Mapping

from .responsibility import Span


@dataclass(frozen=True)
class SourceWrite:
    source: int
    logical_id: str
    lo: int
    hi: int
    klass: str            # replicated | sharded | private


def compile_source_policy(policy: str, responsibilities: Mapping[str, list[Span]],
                          private: Iterable[str] = ()) -> tuple[dict[str, int], list[SourceWrite]]:
    """Returns (logical objects -> bytes, writes)."""
    if policy not in ("simple", "dedup"):
        raise KeyError(f"source policy {policy!r} (simple | dedup)")
    priv = set(private)
    logical: dict[str, int] = {}
    writes: list[SourceWrite] = []
    for oid, spans in responsibilities.items():
        total = max((s.hi for s in spans), default=0)
        if oid in priv:
            for s in spans:
                logical[f"{oid}@{s.source}"] = s.hi - s.lo
                writes.append(SourceWrite(s.source, f"{oid}@{s.source}", 0, s.hi - s.lo, "private"))
            continue
        logical[oid] = total
        whole = all(s.lo == 0 and s.hi == total for s in spans)
        for s in spans:
            if policy == "dedup" and s.replica:
                continue
            writes.append(SourceWrite(s.source, oid, s.lo, s.hi, "replicated" if whole and len(spans) > 1 else "sharded"))
    return logical, writes
