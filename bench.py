#!/usr/bin/env python
"""Headline benchmark: training tokens/s of Llama-3-8B (seq 4096, bf16 + fp32 master
weights, AdamW) under a fixed per-GPU fast-memory budget, through the framework's
public ``Trainer`` API, on N GPUs of one node.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 3 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference, same metric and config

Weak scaling: every GPU processes ``--tokens-per-gpu`` tokens per step (131072 by
default, i.e. 1M tokens per step on 8 GPUs).  Data is synthetic (uniform random
token ids, seed 0) and weights are random-init.  Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

BASELINE_TOK_S = 12618.0     # reference's best published llama3_8b number (1x H100 80GB, seq 1024)

PRESET_BUDGET_GIB = {"llama3_8b": 60.0}


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--preset", default="llama3_8b")
    ap.add_argument("--family", default="llama3")
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=4, help="sequences per grad-accumulation round")
    ap.add_argument("--tokens-per-gpu", type=int, default=131072)
    ap.add_argument("--budget-gib", type=float, default=None)
    ap.add_argument("--dtype-policy", default="bf16_split_master",
                    help="bf16 weights with an exact fp32 master stored split (low halves + bf16 moments as optimizer state)")
    ap.add_argument("--layers", type=int, default=None, help="debug only: cut the model (the result is not a valid bench)")
    ap.add_argument("--kernels", default=None, help="kernel lane override (e.g. baseline)")
    ap.add_argument("--linear-precision", default="bf16", choices=["bf16", "fp8"],
                    help="fp8: e4m3 forward projections (an extra data point; the headline metric is the bf16 run)")
    ap.add_argument("--no-profile", action="store_true", help="plan from roofline seeds instead of measured task costs")
    ap.add_argument("--parallel", default=None, help="fsdp | zero3 | zero1 (default: fsdp when --gpus > 1)")
    ap.add_argument("--plan-only", action="store_true",
                    help="no device: plan the configuration from roofline costs, dry-run the plan against its pools on the "
                         "virtual-time backend and print what is predicted (not a measurement, not the bench line)")
    return ap.parse_args(argv)


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


def bench_ours(a) -> dict:
    import dataclasses
    import torch
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if a.gpus > 1 and world != a.gpus:
        raise SystemExit(f"--gpus {a.gpus} needs WORLD_SIZE={a.gpus} (launch with torch.distributed.run)")
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.ops import cuda as cuda_lane
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    fam = resolve_family(a.family)
    cfg = fam.presets[a.preset]()
    rounds = max(a.tokens_per_gpu // (a.seq_len * a.batch), 1)
    cfg = dataclasses.replace(cfg, seq_len=a.seq_len, batch=a.batch, grad_accum_rounds=rounds, dtype_policy=a.dtype_policy)
    if a.layers:
        cfg = dataclasses.replace(cfg, n_layers=a.layers)
    budget = a.budget_gib if a.budget_gib is not None else PRESET_BUDGET_GIB.get(a.preset, 60.0)
    parallel = a.parallel or ("fsdp" if world > 1 else "solo")
    groups, lower_kwargs = {}, {"resident_params": True}      # weights stay on the device from step to step
    if world > 1:
        from dataflow_b200.parallel.zero import make_dp_group, zero_lower_kwargs
        groups = {"dp": make_dp_group(rank, world, local)}
        lower_kwargs = zero_lower_kwargs(parallel, rank, world)
    hyper = {"lr": 3e-4, "weight_decay": 0.1, "beta1": 0.9, "beta2": 0.95}
    if a.linear_precision != "bf16":
        hyper["linear_precision"] = a.linear_precision
    from dataflow_b200.lowering import resolve_hardware
    # all ranks of the node stream through one host memory: plan with what the host delivers to all of them at once (measured)
    from dataflow_b200.run.scaling import hardware_as_shared
    hw = hardware_as_shared(resolve_hardware(None), world, local)
    tr = Trainer(a.family, cfg, budget_gib=budget, device=local, hyper=hyper, seed=0, kernel_set=a.kernels, hw=hw,
                 profile=not a.no_profile, groups=groups, lower_kwargs=lower_kwargs)
    tokens_step = tr.T * tr.rounds
    vocab = cfg.vocab_size

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    h2d = d2h = 0
    for s in range(a.warmup):
        tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, vocab, rank, s, pin=True), valid_rows=tokens_step * world)
    barrier()
    cuda_lane.LAUNCHES.reset()
    sampler = ClockSampler(local)
    sampler.start()
    data = [synthetic_rounds(cfg, tr.rounds, tr.T, vocab, rank, a.warmup + s, pin=True) for s in range(a.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.perf_counter()
    e0.record()
    dev_us = exposed_us = 0.0
    losses = []
    for s in range(a.steps):
        for r, (tk, tg) in enumerate(data[s]):
            h2d += tr.put_round(r, tk, tg)          # pinned host -> engine store; the engine DMA-copies it to the device
        losses.append(tr.step(None, valid_rows=tokens_step * world))     # reads the loss words back from pinned memory
        d2h += 4 * len(tr.loss_ids)
        dev_us += tr.last_result.makespan_us
        exposed_us += float(tr.last_result.stats.get("exposed_comm_us", 0.0))
    e1.record()
    barrier()
    wall_s = time.perf_counter() - t0
    ev_s = e0.elapsed_time(e1) / 1e3
    clocks = sampler.stop()
    launches = cuda_lane.LAUNCHES.total
    t = torch.tensor([dev_us / 1e6, max(ev_s, wall_s), exposed_us / 1e3], dtype=torch.float64, device="cuda")
    lsum = torch.tensor([losses[-1] if losses else 0.0], dtype=torch.float64, device="cuda")
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        torch.distributed.all_reduce(lsum)          # every rank holds its share of the step's mean loss
    dev_s, e2e_s, exposed_ms = float(t[0]), float(t[1]), float(t[2])
    total_tokens = tokens_step * world * a.steps
    value = total_tokens / dev_s
    res = tr.last_result
    out = {
        "metric": "train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": dev_s / a.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / BASELINE_TOK_S, "dtype": "bf16" if a.linear_precision == "bf16" else "bf16 (fp8 forward projections)",
        "data": "synthetic", "impl": "ours",
        "config": {"model": a.preset + (f"-cut{a.layers}L" if a.layers else ""), "global_batch": tokens_step * world // a.seq_len,
                   "seq_len": a.seq_len, "tokens_per_step": tokens_step * world,
                   "parallelism": parallel if world > 1 else "solo", "fast_budget_gib": budget,
                   "dtype_policy": a.dtype_policy, "optimizer": "adamw", "l2": "inputs_larger_than_L2",
                   "costs": "measured" if tr.measured else "roofline"},
        "clocks": clocks,
        "e2e": {"value": total_tokens / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d // a.steps,
                "d2h_bytes_per_step": d2h // a.steps},
        "gpu_launches": launches,
        # device-timed: what the compute stream spent waiting on parameter gathers / gradient reduce-scatters that run on
        # the communication stream (max over ranks, per step); 0 on one GPU, where nothing is communicated
        "exposed_comm_ms_per_step": exposed_ms / a.steps,
        "loss": float(lsum[0]) if losses else None,
        "plan": {"planner": str(tr.planned.policy), "predicted_ms_per_step": tr.planned.makespan_us / 1e3, "peak_fast_gib": tr.planned.peak_fast_bytes / 2**30,
                 "recompute_layers": len(tr.planned.recompute_levels), "engine_h2d_gb_per_step": res.stats["h2d_bytes"] / 1e9,
                 "engine_d2h_gb_per_step": res.stats["d2h_bytes"] / 1e9, "slab_overflows": res.slab_overflows, "pool": _pool_line(tr),
                 "static_placement": tr.placement is not None,
                 "param_gather": getattr(groups.get("dp"), "gather_mode", None),
                 "host_link_gbs_planned": [round(hw.h2d_gbs, 1), round(hw.d2h_gbs, 1)],
                 "placement_escapes": res.placement_escapes, "pressure_evictions": res.pressure_evictions,
                 "plan_s": tr.plan_s},
        "kernels": {"native_ops": len(tr.K.native_ops()), "lanes": sorted(set(tr.K.describe().values()))},
    }
    if os.environ.get("DFB_BENCH_TRACE") and rank == 0:
        from dataflow_b200.run.trace_report import summarize_trace
        with open(os.environ["DFB_BENCH_TRACE"], "w") as f:
            json.dump({"summary": summarize_trace(tr.program, res), "measured": tr.measured,
                       "plan_transfer": tr.planned.transfer}, f, indent=1)
    tr.close()
    if world > 1:
        torch.distributed.destroy_process_group()
    return out if rank == 0 else {}


def _pool_line(tr) -> dict:
    """How the fast pool is backed, and (vmm mode) how many pages it mapped and moved so far."""
    try:
        st = tr.session.native.fast_pool_stats()
    except Exception:       # noqa: BLE001
        return {"mode": getattr(tr, "pool_mode", "slab")}
    out = {k: (int(v) if not isinstance(v, str) else v) for k, v in st.items() if k in ("mode", "maps", "reclaims", "phys_pages", "held_pages")}
    try:
        # overflows by pool since the run began, and what the dry run of the plan said the pools would be asked for
        out["fast_overflows_total"] = int(st.get("overflows", 0))
        out["backing_overflows_total"] = int(tr.session.native.backing_pool_stats().get("overflows", 0))
        d = getattr(tr, "pool_demand", None)
        if d is not None:
            out["dry_run"] = {"fast_overflows_per_step": d.fast_overflows, "backing_peak_gib": round(d.backing_peak / 2 ** 30, 3)}
    except Exception:       # noqa: BLE001
        pass
    return out


def plan_only(a) -> dict:
    """The planning half of the bench on the CPU: the configuration ``bench_ours`` would run, planned from the hardware row's
    roofline costs (a device run plans from measured task costs), then the pool fitting a device run does before its first
    step.  Says what the plan predicts and what the pools would be asked for; measures nothing."""
    import dataclasses
    from types import SimpleNamespace
    from dataflow_b200.lowering import resolve_hardware
    from dataflow_b200.lowering.planning import DEFAULT_PROGRAM_LEEWAY_BYTES
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.run.driver import Trainer, plan_at_budget
    from dataflow_b200.runtime.pool_demand import dry_run_pools
    fam = resolve_family(a.family)
    cfg = fam.presets[a.preset]()
    rounds = max(a.tokens_per_gpu // (a.seq_len * a.batch), 1)
    cfg = dataclasses.replace(cfg, seq_len=a.seq_len, batch=a.batch, grad_accum_rounds=rounds, dtype_policy=a.dtype_policy)
    if a.layers:
        cfg = dataclasses.replace(cfg, n_layers=a.layers)
    budget_gib = a.budget_gib if a.budget_gib is not None else PRESET_BUDGET_GIB.get(a.preset, 60.0)
    budget = int(budget_gib * (1 << 30))
    world = max(a.gpus, 1)
    parallel = a.parallel or ("fsdp" if world > 1 else "solo")
    lower_kwargs = {"resident_params": True}
    if world > 1:
        from dataflow_b200.parallel.zero import zero_lower_kwargs
        lower_kwargs = zero_lower_kwargs(parallel, 0, world)
    hw = resolve_hardware("b200").shared(world)
    planned = plan_at_budget(fam, cfg, budget, hw, lower_kwargs=lower_kwargs)
    sizes = {}
    for o in planned.program.initial_objects:
        sizes.setdefault(o.id, o.size_bytes)
    for t in planned.program.tasks:
        for out in t.outputs:
            if out.location == "backing" and out.id.startswith("loss_"):
                sizes[out.id] = out.size_bytes
    pool = planned.object_capacity + min(DEFAULT_PROGRAM_LEEWAY_BYTES * 3 // 4, 1 << 30)
    keep = any(loc == "fast" for loc in planned.program.final_locations.values())
    ledger = max(planned.peak_backing_bytes - sum(sizes.values()), 0) + (64 << 20)
    first = dry_run_pools(planned.program, sizes, pool, backing_capacity=ledger, keep_resident=keep, dispatch_ahead=2)
    stub = SimpleNamespace(program=planned.program, planned=planned, fam=fam, hw=hw, verbose=False, pool_demand=None)
    backing = Trainer._fit_pools(stub, cfg, sizes, pool, ledger, keep, budget, True, None, None, lower_kwargs, replan=world == 1)
    final = dry_run_pools(stub.program, sizes, pool, backing_capacity=backing, keep_resident=keep, dispatch_ahead=2, steps=3)
    tokens = a.tokens_per_gpu // (a.seq_len * a.batch) * a.seq_len * a.batch
    gib = 2 ** 30
    return {"plan_only": True, "note": "predicted from roofline costs on the CPU; not a measurement",
            "config": {"model": a.preset, "seq_len": a.seq_len, "tokens_per_gpu": tokens, "rounds": rounds, "budget_gib": budget_gib,
                       "parallelism": parallel if world > 1 else "solo", "n_gpus": world},
            "first_plan": {"policy": planned.policy, "predicted_ms_per_step": planned.makespan_us / 1e3, "peak_fast_gib": planned.peak_fast_bytes / gib,
                           "pools_from_the_plans_ledger": {"fast_gib": pool / gib, "backing_gib": ledger / gib,
                                                           "fast_overflows_per_step": first.fast_overflows, "backing_overflows_per_step": first.backing_overflows}},
            "fitted": {"policy": stub.planned.policy, "replanned": stub.planned is not planned, "predicted_ms_per_step": stub.planned.makespan_us / 1e3,
                       "predicted_tokens_per_s_per_gpu": tokens / stub.planned.makespan_us * 1e6, "peak_fast_gib": stub.planned.peak_fast_bytes / gib,
                       "pools": {"fast_gib": pool / gib, "backing_gib": backing / gib, "fast_overflows_per_step": final.fast_overflows,
                                 "backing_overflows_per_step": final.backing_overflows}}}


def main(argv=None) -> int:
    a = parse_args(argv)
    if a.plan_only:
        print(json.dumps(plan_only(a)), flush=True)
        return 0
    if a.impl == "reference":
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from baseline.reference_arm import run_reference_arm
        out = run_reference_arm(a)
    else:
        out = bench_ours(a)
    if out:
        print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
