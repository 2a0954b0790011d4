"""Replay a measured step through the simulator.

``replay_program`` keeps the plan (task order and transfer directives) but replaces every task's runtime with the
duration the engine MEASURED for it; simulating that program gives the step time the schedule would reach with zero
dispatch overhead and ideal lanes.  ``replay_gap_pct`` is the measured makespan's excess over that: the share of a
step that is scheduling overhead (launch gaps, copy-lane contention) rather than kernel time.
Reference role: ``src/dataflow_training/lowering/replay.py:17,57``.
"""
from __future__ import annotations

from dataclasses import replace
from typing import Mapping

from ..core.convert import to_sim_chain
from ..sim.simulator import run as simulate


def measured_durations(trace) -> dict[str, float]:
    """Task id -> measured compute-lane duration (µs) from a run trace."""
    return {iv.name: iv.end_us - iv.start_us for iv in trace.by_track("compute")}


def replay_program(program, durations_us: Mapping[str, float], *, h2d_bytes_per_us: float | None = None,
                   d2h_bytes_per_us: float | None = None):
    """The same annotated program with measured task runtimes (and, optionally, measured link bandwidths)."""
    tasks = tuple(replace(t, runtime_us=float(durations_us.get(t.id, t.runtime_us))) for t in program.tasks)
    kw = {}
    if h2d_bytes_per_us:
        kw["bandwidth_from_slow"] = int(h2d_bytes_per_us)
    if d2h_bytes_per_us:
        kw["bandwidth_to_slow"] = int(d2h_bytes_per_us)
    return replace(program, tasks=tasks, **kw)


def replay_makespan_us(program, durations_us: Mapping[str, float], **bw) -> float:
    chain = to_sim_chain(replay_program(program, durations_us, **bw))
    if (program.metadata or {}).get("workspace_accounting") == "external":
        # the plan's capacity is the object pool alone; scratch lives outside it
        chain = replace(chain, tasks=[replace(t, workspace_bytes=0) for t in chain.tasks])
    return float(simulate(chain, validate=False).makespan)


def replay_gap_pct(program, result, *, use_measured_links: bool = False) -> dict[str, float]:
    """``result``: an engine run of ``program`` with its interval trace."""
    dur = measured_durations(result.trace)
    bw = {}
    if use_measured_links:
        h, d = result.trace.busy_us("from_slow"), result.trace.busy_us("to_slow")
        if h > 0 and result.stats.get("h2d_bytes"):
            bw["h2d_bytes_per_us"] = result.stats["h2d_bytes"] / h
        if d > 0 and result.stats.get("d2h_bytes"):
            bw["d2h_bytes_per_us"] = result.stats["d2h_bytes"] / d
    ideal = replay_makespan_us(program, dur, **bw)
    measured = float(result.makespan_us)
    return {"measured_us": measured, "replay_us": ideal, "compute_us": float(sum(dur.values())),
            "gap_pct": 100.0 * (measured - ideal) / ideal if ideal else 0.0}
