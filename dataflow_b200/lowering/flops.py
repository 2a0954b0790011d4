"""FLOP accounting of a lowered program from the ``cost_subops`` stamped on its tasks.

*Effective* FLOPs are the ones the model needs (forward, backward, head, optimizer matmuls); *hardware* FLOPs add the
recomputed forwards the plan chose.  Attention sub-ops (tagged ``efficiency: attention*``) are reported on their own
so a step's matmul and attention shares can be read off.  ``completeness`` lists compute tasks that carry no
sub-ops (a family whose lowering forgot to stamp them would silently under-report).
Reference role: ``src/dataflow_training/lowering/flops.py:52-168`` (``flop_report``).
"""
from __future__ import annotations

from typing import Any

PHASES = ("fwd", "recompute", "bwd", "head", "optimizer", "other")
_NO_FLOPS_KEYS = ("prologue_round", "embed_fwd", "embed_bwd", "optimizer_embed", "optimizer_head", "zero_gather", "grad_rs",
                  "grad_rs_join", "optimizer_block", "optimizer_local")


def task_phase(task) -> str:
    k = task.compute_block_key or ""
    if k.endswith("_recompute"):
        return "recompute"
    if k.endswith("_fwd"):
        return "fwd"
    if k.endswith("_bwd"):
        return "bwd"
    if k.startswith("head"):
        return "head"
    if k.startswith("optimizer"):
        return "optimizer"
    return "other"


def flop_report(program, makespan_us: float | None = None) -> dict[str, Any]:
    by_phase = {p: {"flops": 0.0, "attention_flops": 0.0, "memory_bytes": 0.0, "tasks": 0} for p in PHASES}
    missing = []
    for t in program.tasks:
        ph = by_phase[task_phase(t)]
        ph["tasks"] += 1
        subs = t.metadata.get("cost_subops") if t.metadata else None
        if not subs:
            if t.compute_block_key and not any(t.compute_block_key.startswith(k) for k in _NO_FLOPS_KEYS) and not t.host:
                missing.append(t.id)
            continue
        for s in subs:
            f = float(s.get("flops", 0.0))
            ph["flops"] += f
            if str(s.get("efficiency", "")).startswith("attention"):
                ph["attention_flops"] += f
            ph["memory_bytes"] += float(s.get("memory_bytes", 0.0))
    hardware = sum(p["flops"] for p in by_phase.values())
    effective = hardware - by_phase["recompute"]["flops"]
    tokens = int((program.metadata or {}).get("tokens_per_step", 0))
    out = {"effective_flops": effective, "hardware_flops": hardware, "recompute_flops": by_phase["recompute"]["flops"],
           "attention_flops": sum(p["attention_flops"] for p in by_phase.values()), "tokens_per_step": tokens,
           "effective_flops_per_token": effective / tokens if tokens else 0.0, "by_phase": by_phase, "completeness": missing}
    if makespan_us:
        out["effective_tflops"] = effective / makespan_us / 1e6
        out["hardware_tflops"] = hardware / makespan_us / 1e6
    return out


def print_table(report: dict[str, Any]) -> str:
    lines = [f"{'phase':<10} {'tasks':>6} {'GFLOP':>12} {'attn GFLOP':>12} {'GB moved':>10}"]
    for name, p in report["by_phase"].items():
        if p["tasks"]:
            lines.append(f"{name:<10} {p['tasks']:>6} {p['flops'] / 1e9:>12.1f} {p['attention_flops'] / 1e9:>12.1f} {p['memory_bytes'] / 1e9:>10.2f}")
    lines.append(f"effective {report['effective_flops'] / 1e12:.3f} TFLOP  hardware {report['hardware_flops'] / 1e12:.3f} TFLOP"
                 + (f"  -> {report['effective_tflops']:.1f} / {report['hardware_tflops']:.1f} TFLOP/s" if "effective_tflops" in report else ""))
    return "\n".join(lines)
