"""What one rank of a training job does: resolve the config, build the trainer (plan, init or resume), run the
loop, save the result (rank 0).  Entry of ``torch.distributed.run`` for multi-GPU jobs and called in-process for
solo runs."""
from __future__ import annotations

import argparse
import dataclasses
import os
import sys
from typing import Any

from .conductor import RunSpec
from .driver import RunResult, Trainer


def build_cfg(spec: RunSpec):
    from .presets import resolve_preset
    family, cfg = resolve_preset(spec.preset)
    known = {f.name for f in dataclasses.fields(cfg)}
    bad = set(spec.overrides) - known
    if bad:
        raise KeyError(f"preset {spec.preset!r} has no config fields {sorted(bad)}")
    return family, dataclasses.replace(cfg, **spec.overrides)


def run_rank(spec: RunSpec, log=print) -> RunResult:
    from ..data.pipeline import pipeline_from_args
    from .checkpointing import load_checkpoint, resolve_resume
    from .loop import train_loop
    from .recipe import Recipe
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1)) if spec.world > 1 else 1
    local = int(os.environ.get("LOCAL_RANK", 0))
    device = None if spec.device is None else (local if world > 1 else spec.device)
    if device is not None and spec.devices:
        if len(spec.devices) != max(world, 1):
            raise ValueError(f"{len(spec.devices)} devices named for a job of {world} ranks")
        device = int(spec.devices[local])
    groups: dict[str, Any] = {}
    lower_kwargs: dict[str, Any] = {}
    if spec.backend not in ("auto", "peer", "nccl"):
        raise ValueError(f"--backend is auto, peer or nccl, not {spec.backend!r}")
    if spec.backend == "peer" and device is None:
        raise ValueError("--backend peer moves data with kernels over peer GPU memory: it needs --device on GPUs (CPU ranks use nccl / auto)")
    lane = "collective" if spec.backend == "nccl" else ("p2p" if spec.backend == "peer" else None)
    if spec.refresh_profiles:
        os.environ["DATAFLOW_PROFILE_REFRESH"] = "1"
    if world > 1:
        import torch
        import torch.distributed as dist
        import datetime
        # a rank that died is noticed by the others when their next collective runs out of time
        timeout = datetime.timedelta(seconds=float(os.environ.get("DATAFLOW_PG_TIMEOUT_S", "1800")))
        if device is None:
            dist.init_process_group("gloo", timeout=timeout)
        else:
            torch.cuda.set_device(device)
            dist.init_process_group("nccl", device_id=torch.device("cuda", device), timeout=timeout)
        if spec.parallel not in ("tp", "ep"):
            from ..parallel.zero import make_dp_group, zero_lower_kwargs
            # plain data parallelism needs no peer-mapped slab: its one collective per optimizer task is a library all-reduce
            groups = {"dp": make_dp_group(rank, world, device, "collective" if spec.parallel in ("co", "dp") else lane)}
            lower_kwargs = zero_lower_kwargs(spec.parallel, rank, world)
            if spec.parallel in ("co", "dp") and spec.resident_params and device is not None:
                lower_kwargs = {"resident_params": True}
    elif spec.resident_params:
        lower_kwargs = {"resident_params": True}
    family, cfg = build_cfg(spec)
    data_world = world
    if spec.rounds:
        if world <= 1 or spec.parallel not in ("co", "dp") or len(spec.rounds) != world:
            raise ValueError("--rounds a,b,... gives every rank its own number of rounds: it needs --parallel co and one entry per rank")
        cfg = dataclasses.replace(cfg, grad_accum_rounds=int(spec.rounds[rank]))
    if world > 1 and spec.parallel == "tp":
        # tensor + sequence parallelism: the dense llama block split over the ranks (family tp_mlp)
        from ..parallel.tp import TpGroup
        if family not in ("llama3", "tp_mlp"):
            raise ValueError(f"--parallel tp covers the dense llama block (llama3 / tp_mlp presets), not {family!r}")
        tp = int(spec.tp_size or world)
        if tp < 2 or world % tp:
            raise ValueError(f"--tp-size {tp} does not divide the job's {world} ranks into tensor-parallel groups")
        dp = world // tp
        family, cfg = "tp_mlp", dataclasses.replace(cfg, tp=tp, family="tp_mlp")
        from ..models.families import resolve_family
        d = resolve_family(family).derive_dims(cfg)
        tp_pg = dp_pg = None
        if dp > 1:
            # a dp x tp mesh (tp the fastest-varying axis): the scheme names every rank's partners; every rank creates every
            # subgroup, in the same order
            import torch.distributed as dist
            from ..distributed.parallelism import scheme_from_flags
            scheme = scheme_from_flags(world, opt_shard="co", tp=tp)
            for axis in ("tp", "dp"):
                for members in sorted({tuple(scheme.group_members(axis, r)) for r in range(world)}):
                    pg = dist.new_group(list(members))
                    if rank in members:
                        tp_pg, dp_pg = (pg, dp_pg) if axis == "tp" else (tp_pg, pg)
        groups = {"tp": TpGroup(rank % tp, tp, device, max_rows=d.Ts, max_k=d.d, max_n=d.d, lane=lane, pg=tp_pg)}
        if dp > 1:
            from ..parallel.zero import make_dp_group
            groups["dp"] = make_dp_group(rank // tp, dp, device, "collective", pg=dp_pg)
        lower_kwargs = {"resident_params": True} if spec.resident_params and device is not None else {}
        data_world = dp
    elif world > 1 and spec.parallel == "ep":
        # expert parallelism: experts split over the ranks, everything else data-parallel
        from ..models.families import resolve_family
        from ..parallel.ep import ep_group_for
        if "ep" not in {f.name for f in dataclasses.fields(cfg)}:
            raise ValueError(f"--parallel ep needs a mixture-of-experts preset, {spec.preset!r} has no experts to split")
        ep = int(spec.ep_size or world)
        if ep < 2 or world % ep:
            raise ValueError(f"--ep-size {ep} does not divide the job's {world} ranks into expert-parallel groups")
        cfg = dataclasses.replace(cfg, ep=ep)
        ep_pg = dp_pg = None
        if world > ep:
            # a dp x ep mesh (ep the fastest-varying axis): consecutive ranks share one copy of the experts; ranks with the
            # same place in their groups hold the same experts and sum those gradients among themselves
            import torch.distributed as dist
            from ..distributed.parallelism import scheme_from_flags
            scheme = scheme_from_flags(world, opt_shard="co", ep=ep)
            for axis in ("ep", "dp"):
                for members in sorted({tuple(scheme.group_members(axis, r)) for r in range(world)}):
                    pg = dist.new_group(list(members))
                    if rank in members:
                        ep_pg, dp_pg = (pg, dp_pg) if axis == "ep" else (ep_pg, pg)
        try:
            groups = {"ep": ep_group_for(resolve_family(family), cfg, rank % ep, ep, device, lane, pg=ep_pg)}
        except ValueError as e:
            raise ValueError(f"--parallel ep needs a mixture-of-experts preset, {spec.preset!r} is dense ({e})") from None
        if world > ep:
            from ..parallel.zero import make_dp_group
            groups["dp"] = make_dp_group(rank // ep, world // ep, device, "collective", pg=dp_pg)
        lower_kwargs = {"resident_params": True} if spec.resident_params and device is not None else {}
    recipe = Recipe(**{"total_steps": spec.steps, **spec.recipe})
    say = log if rank == 0 else (lambda *a, **k: None)
    hw = None
    if device is not None and world > 1:
        from ..lowering import resolve_hardware
        from .scaling import hardware_as_shared
        hw = hardware_as_shared(resolve_hardware(None), world, device)          # what the host gives all ranks at once
    tr = Trainer(family, cfg, budget_gib=spec.budget_gib, device=device, hyper=recipe.hyper(), seed=spec.seed,
                 kernel_set=spec.kernels, recompute=spec.recompute, profile=spec.profile and device is not None,
                 groups=groups, lower_kwargs=lower_kwargs or None, hw=hw)
    if spec.backing_budget_gib is not None and tr.store.total > spec.backing_budget_gib * 2 ** 30:
        need = tr.store.total / 2 ** 30
        tr.close()
        raise ValueError(f"the run's host store needs {need:.2f} GiB of pinned memory, --backing-budget allows {spec.backing_budget_gib:g}")
    if spec.warm_profiles:
        say(f"task costs measured and cached ({tr.program.metadata.get('costs', 'roofline seeds')}); --warm-profiles stops here")
        tr.close()
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
        from .driver import RunResult
        return RunResult(losses=[], tokens_per_step=tr.T * tr.rounds * world, meta={"warm_profiles": True})
    say(f"plan: {tr.planned.policy}, predicted {tr.planned.makespan_us / 1e3:.1f} ms/step, peak fast "
        f"{tr.planned.peak_fast_bytes / 2 ** 30:.2f} GiB, planned in {tr.plan_s:.1f} s")
    # the job-wide pipeline: every rank packs all rounds of the step and keeps its own
    if world > 1 and (spec.parallel in ("co", "dp") or (spec.parallel == "tp" and "dp" in groups)):
        from ..parallel.zero import replicate_gradients
        replicate_gradients(tr)
    if spec.parallel == "ep" and "dp" in groups:
        from ..parallel.ep import sum_expert_gradients_over_replicas
        sum_expert_gradients_over_replicas(tr)
    total_rounds = sum(spec.rounds) if spec.rounds else cfg.grad_accum_rounds * data_world
    wide = dataclasses.replace(cfg, grad_accum_rounds=total_rounds)
    factory = pipeline_from_args(wide, spec.data, policy=spec.packing_policy, allow_round_split=spec.allow_round_split,
                                 capture=spec.capture if rank == 0 else None)
    start, cursor, losses = 0, None, []
    sdir = resolve_resume(spec.resume, spec.checkpoint_dir)
    if sdir:
        rec = load_checkpoint(tr, sdir)
        payload = rec.get("client_payload") or {}
        start, cursor, losses = int(rec["step"]), payload.get("cursor"), list(payload.get("losses") or [])
        say(f"resumed from {sdir} at step {start}")
    launch = {"argv": spec.argv, "resolved": {"preset": spec.preset, "seed": spec.seed, "world": world,
                                              "parallel": spec.parallel if world > 1 else "solo", **spec.overrides},
              "data": factory.describe(), "env": _env_facts()}
    from .profiling import ProfileWindow
    window = ProfileWindow(spec.prof_dir, spec.profile_start_before_step, spec.profile_stop_after_step, rank)
    try:
        res = train_loop(tr, factory, spec.steps, cursor=cursor, start_step=start, losses=losses, rank_rounds=spec.rounds,
                         on_step=_host_fault_plan(rank), window=window,
                         checkpoint_every=spec.checkpoint_every, checkpoint_dir=spec.checkpoint_dir,
                         keep_last=spec.checkpoint_keep_last, checkpoint_redundancy=spec.checkpoint_redundancy, seed=spec.seed, launch=launch, log=say)
    finally:
        tr.close()
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
    res.meta["launch"] = launch
    if window.written:
        res.meta["traces"] = list(window.written)
    if spec.out and rank == 0:
        res.save(spec.out)
    return res


def _host_fault_plan(rank: int):
    """Host-side fault injection for failure-detection drills: ``DATAFLOW_FAULT_PLAN="rank=1,step=2,kind=raise"`` makes that
    rank raise (or ``kind=exit``: leave without a word) right after the named step, between steps, with nothing of its own
    in flight.  ``once=<path>``: the fault fires only while that marker file does not exist and creates it (a restarted job
    then runs through).  Nothing is injected on a device."""
    plan = os.environ.get("DATAFLOW_FAULT_PLAN")
    if not plan:
        return None
    kv = dict(item.split("=", 1) for item in plan.split(","))
    if int(kv.get("rank", -1)) != rank:
        return None
    at, kind, once = int(kv.get("step", 1)), kv.get("kind", "raise"), kv.get("once")

    def on_step(step, loss, packed):
        if step == at:
            if once:
                if os.path.exists(once):
                    return
                open(once, "w").close()
            if kind == "exit":
                os._exit(17)
            raise RuntimeError(f"fault plan: rank {rank} fails after step {step}")
    return on_step


def _env_facts() -> dict:
    import torch
    return {"torch": torch.__version__, "cuda": torch.version.cuda, "python": sys.version.split()[0]}


def failure_kind(exc: BaseException) -> str:
    """``device``: the GPU context or a fused kernel reported the failure (a CUDA error, a kernel's error word) — running
    the same job again would run the same faulty work on a shared GPU.  ``timeout``: a collective gave up waiting for a
    peer.  ``host``: anything else (an exception in Python code, a fault plan)."""
    from ..parallel.zero import CommTimeout
    text = f"{type(exc).__name__}: {exc}"
    if isinstance(exc, CommTimeout):
        return "timeout"
    low = text.lower()
    if any(k in low for k in ("cuda error", "acceleratorerror", "illegal memory", "illegal instruction", "misaligned address",
                              "device-side assert", "unspecified launch failure", "error word", "kernel gave up")):
        return "device"
    if "timeout" in low or "timed out" in low:
        return "timeout"
    return "host"


def failure_marker(out: str, rank: int) -> str:
    return f"{out}.failure.rank{rank}"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--spec", required=True)
    a = ap.parse_args(argv)
    spec = RunSpec.from_json(a.spec)
    try:
        run_rank(spec)
    except BaseException as e:          # noqa: BLE001 - classified for the conductor, then re-raised
        if spec.out and not isinstance(e, (SystemExit, KeyboardInterrupt)):
            import json
            with open(failure_marker(spec.out, int(os.environ.get("RANK", 0))), "w") as f:
                json.dump({"kind": failure_kind(e), "message": f"{type(e).__name__}: {e}"[:2000]}, f)
        raise
    return 0


if __name__ == "__main__":
    sys.exit(main())
