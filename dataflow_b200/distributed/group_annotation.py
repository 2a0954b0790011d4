"""Stamp a lowered program with the groups and shard facts of a scheme: every task that communicates gets
``comm_groups`` (purpose -> group name) and its ``block_params`` learn the rank's coordinates; tensor-parallel
schemes swap the compute key prefix of sharded blocks to ``tp_``.
Role parity: reference ``src/dataflow_training/distributed/group_annotation.py:45-140``.
"""
from __future__ import annotations

from dataclasses import replace
from typing import Mapping

from ..core import Program
from .parallelism import ParallelismScheme

COMM_KEYS = ("optimizer_", "param_gather", "tp_", "ep_", "moe_")


def annotate_groups(program: Program, scheme: ParallelismScheme, rank: int,
                    group_names: Mapping[str, str] | None = None) -> Program:
    """``group_names``: axis name -> peer group name (default: the axis name)."""
    if not scheme.axes:
        return program
    names = {a.name: (group_names or {}).get(a.name, a.name) for a in scheme.axes}
    coords = scheme.coords(rank)
    shard = {a.name: {"rank": coords[a.name], "world": a.size, "kind": a.kind,
                      **({"responsibility": a.responsibility} if a.kind == "dp" else {}),
                      **({"sequence_parallel": a.sequence_parallel} if a.kind == "tp" else {})} for a in scheme.axes}
    tp = scheme.axis("tp")
    tasks = []
    for t in program.tasks:
        key = t.compute_block_key or ""
        communicates = any(key.startswith(k) for k in COMM_KEYS) or (tp is not None and key.startswith("block"))
        if not communicates:
            tasks.append(t)
            continue
        cg = {**dict(t.comm_groups), **{a.kind: names[a.name] for a in scheme.axes}}
        bp = {**dict(t.block_params), "axes": shard}
        if tp is not None and key.startswith("block") and not key.startswith("tp_"):
            key = "tp_" + key
        tasks.append(replace(t, comm_groups=cg, block_params=bp, compute_block_key=key))
    meta = {**dict(program.metadata or {}), "scheme": scheme.to_dict(), "rank": rank}
    return replace(program, tasks=tuple(tasks), metadata=meta)
