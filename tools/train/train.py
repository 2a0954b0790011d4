#!/usr/bin/env python
"""The training tool.

    train.py train     --preset llama3_8b --steps 100 --fast-budget 60 [--gpus 8] [--data SPEC] [--checkpoint-every N ...]
    train.py reference --preset tiny --steps 20          # the pure-torch twin on the same data (CPU, fp32)
    train.py smoke     [--preset tiny] [--device cpu]    # a few steps end to end, asserts a healthy curve
    train.py parity    --preset tiny --steps 8           # engine vs twin from identical init and data
    train.py scaling   --preset l3_125m --gpus 1,2,4     # tokens/s per world size + fit
    train.py peek      CHECKPOINT_DIR                    # what a checkpoint holds
    train.py compare   A.json B.json [--band bf16]       # two saved curves

Role parity: reference ``tools/train/train.py:112-457`` (same subcommands and flag vocabulary; ``--gpus`` replaces
the topology / group flags because ranks here are processes of one node, one per GPU).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def add_run_flags(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--preset", default="llama3:tiny", help="preset name or family:preset")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--peak-lr", type=float, default=3e-4)
    ap.add_argument("--min-lr", type=float, default=None)
    ap.add_argument("--warmup-steps", type=int, default=0)
    ap.add_argument("--muon-lr", type=float, default=None)
    ap.add_argument("--opt", default=None, help="adamw | muon | sgd | sgdm")
    ap.add_argument("--ga-rounds", type=int, default=None)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--max-seq-len", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--dtype-policy", default=None)
    ap.add_argument("--linear-precision", default=None, choices=["bf16", "fp8"],
                    help="operand precision of the dense forward projections (fp8: e4m3 with per-row / per-column scales)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--fast-budget", type=float, default=None, help="device memory budget in GiB")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--device", default="0", help="CUDA ordinal, or 'cpu'")
    ap.add_argument("--opt-shard", "--parallel", dest="opt_shard", default="fsdp", choices=["fsdp", "zero3", "zero1", "zero1rs", "co", "tp", "ep"],
                    help="how --gpus N ranks split the job: fsdp / zero3 / zero1 shard parameters and optimizer state over data-parallel "
                         "ranks; co = plain data parallelism (replicas, gradients all-reduced); tp = tensor + sequence parallel llama "
                         "blocks; ep = experts split over the ranks (MoE presets)")
    ap.add_argument("--topology", default=None, help="topology file (TOML: [hosts.*], [groups.*]); with --group it names the ranks' devices")
    ap.add_argument("--group", default=None, help="group of the topology to run on (default: its only group)")
    ap.add_argument("--tp-size", type=int, default=None,
                    help="with --parallel tp: ranks per tensor-parallel group; --gpus N then runs N / tp-size data-parallel replicas of it")
    ap.add_argument("--vocab-parallel", action="store_true",
                    help="with --parallel tp: split the output projection's vocabulary columns over the group (softmax statistics exchanged)")
    ap.add_argument("--ep-size", type=int, default=None,
                    help="with --parallel ep: ranks per expert-parallel group; --gpus N then runs N / ep-size replicas of the experts")
    ap.add_argument("--tp-mlp", action="store_true", help="same as --parallel tp (the reference's flag name)")
    ap.add_argument("--backend", default="auto", choices=["auto", "peer", "nccl"],
                    help="how the ranks exchange data: peer = kernels over peer memory (default on GPUs), nccl = library collectives")
    ap.add_argument("--backing-budget", type=float, default=None, help="pinned host memory the run may use, GiB")
    ap.add_argument("--prof-dir", default=None, help="write the engine trace of every step of the profile window here")
    ap.add_argument("--profile-start-before-step", type=int, default=0, help="first step (1-indexed) of the profile window")
    ap.add_argument("--profile-stop-after-step", type=int, default=0, help="last step of the profile window")
    ap.add_argument("--warm-profiles", action="store_true", help="measure and cache the task costs, then stop")
    ap.add_argument("--refresh-profiles", action="store_true", help="measure task costs again even if cached")
    ap.add_argument("--rounds", default=None, help="weighted data parallelism with --parallel co: rounds per rank, e.g. 6,2")
    ap.add_argument("--kernels", default=None, help="kernel lane: sm100 | baseline | eager")
    ap.add_argument("--profile", action="store_true", help="plan from measured task costs")
    ap.add_argument("--no-recompute", action="store_true")
    ap.add_argument("--no-resident-params", action="store_true")
    ap.add_argument("--checkpoint-every", type=int, default=0)
    ap.add_argument("--checkpoint-dir", default=None)
    ap.add_argument("--checkpoint-keep-last", type=int, default=None)
    ap.add_argument("--checkpoint-redundancy", type=int, default=None,
                    help="how many ranks write their copy of replicated objects (default: all, which also checks them for drift)")
    ap.add_argument("--launcher", default="process", choices=["process", "fleet"],
                    help="process: one rank per process under torch.distributed.run (fused peer-memory lanes); fleet: one dataflowd "
                         "daemon per rank driven by this process over unix sockets (replicas, --opt-shard co)")
    ap.add_argument("--max-restarts", type=int, default=0,
                    help="relaunch a failed multi-rank job from its newest complete checkpoint, up to this many times")
    ap.add_argument("--resume", default=None, help="step directory, checkpoint root, or 'latest'")
    ap.add_argument("--data", default=None, help="scheme:main[,k=v...] (synthetic | shards | jsonl | txt | parquet | capture)")
    ap.add_argument("--packing-policy", default="ffd", choices=["ffd", "greedy"])
    ap.add_argument("--allow-round-split", action="store_true")
    ap.add_argument("--capture", default=None)
    ap.add_argument("--out", default=None, help="write the run curve JSON here")


def ranks_from_topology(path: str, group: str | None):
    """(world, CUDA ordinal of every rank, backend) of a topology group.  One job runs on ONE box here (the ranks talk through
    peer memory and NCCL over NVLink), so every member must sit on a local host."""
    from dataflow_b200.distributed.topology import load_topology
    topo = load_topology(path)
    g = topo.group(group)
    far = [m.key for m in g.members if not topo.host_of(m).local]
    if far:
        raise SystemExit(f"group {g.name!r} names remote members {far}: a job spans one box (cross-box lanes are not built)")
    return g.world, [int(m.device) for m in g.members], g.backend


def spec_from_args(a, argv):
    from dataflow_b200.run.conductor import RunSpec
    devices = None
    if a.topology:
        a.gpus, devices, backend = ranks_from_topology(a.topology, a.group)
        if a.backend == "auto" and backend in ("peer", "nccl"):
            a.backend = backend
    ov = {}
    for flag, fieldname in (("ga_rounds", "grad_accum_rounds"), ("batch", "batch"), ("max_seq_len", "seq_len"),
                            ("layers", "n_layers"), ("dtype_policy", "dtype_policy"), ("opt", "optimizer")):
        v = getattr(a, flag)
        if v is not None:
            ov[fieldname] = v
    if a.vocab_parallel:
        ov["vocab_parallel"] = True
    recipe = {"peak_lr": a.peak_lr, "min_lr": a.min_lr if a.min_lr is not None else a.peak_lr * 0.1,
              "warmup_steps": a.warmup_steps}
    if a.muon_lr is not None:
        recipe["muon_lr"] = a.muon_lr
    if a.linear_precision is not None:
        recipe["linear_precision"] = a.linear_precision
    if a.opt:
        recipe["optimizer"] = a.opt
    return RunSpec(preset=a.preset, steps=a.steps, overrides=ov, recipe=recipe, data=a.data, packing_policy=a.packing_policy,
                   allow_round_split=a.allow_round_split, capture=a.capture, budget_gib=a.fast_budget,
                   device=None if a.device == "cpu" else int(a.device), world=a.gpus, parallel="tp" if a.tp_mlp else a.opt_shard, tp_size=a.tp_size, ep_size=a.ep_size, rounds=[int(x) for x in a.rounds.split(",")] if a.rounds else None, seed=a.seed,
                   profile=a.profile or a.warm_profiles or a.refresh_profiles, recompute=not a.no_recompute, kernels=a.kernels,
                   backend=a.backend, devices=devices, backing_budget_gib=a.backing_budget, prof_dir=a.prof_dir,
                   profile_start_before_step=a.profile_start_before_step, profile_stop_after_step=a.profile_stop_after_step,
                   warm_profiles=a.warm_profiles, refresh_profiles=a.refresh_profiles,
                   resident_params=not a.no_resident_params, checkpoint_every=a.checkpoint_every,
                   checkpoint_dir=a.checkpoint_dir, checkpoint_keep_last=a.checkpoint_keep_last, checkpoint_redundancy=a.checkpoint_redundancy, resume=a.resume, max_restarts=a.max_restarts, out=a.out,
                   launcher=a.launcher, argv=list(argv))


def cmd_train(a, argv) -> int:
    from dataflow_b200.run.conductor import run
    res = run(spec_from_args(a, argv))
    print(f"done: {len(res.losses)} steps, last loss {res.losses[-1]:.4f}, {res.tokens_per_s:,.0f} tok/s" if res.losses else "no steps ran")
    return 0


def _twin_setup(a, argv):
    import dataclasses
    from dataflow_b200.data.pipeline import pipeline_from_args
    from dataflow_b200.run.rank_main import build_cfg
    from dataflow_b200.run.recipe import Recipe
    spec = spec_from_args(a, argv)
    family, cfg = build_cfg(spec)
    recipe = Recipe(**{"total_steps": spec.steps, **spec.recipe})
    factory = pipeline_from_args(cfg, spec.data, policy=spec.packing_policy, allow_round_split=spec.allow_round_split)
    return spec, family, cfg, recipe, factory


def cmd_reference(a, argv) -> int:
    from dataflow_b200.run.driver import Trainer
    from dataflow_b200.run.loop import reference_loop
    spec, family, cfg, recipe, factory = _twin_setup(a, argv)
    # identical init: build the engine's initial values on the CPU store and bridge them into the twin
    tr = Trainer(family, cfg, budget_gib=None, device=None, hyper=recipe.hyper(), seed=spec.seed, recompute=False)
    try:
        res = reference_loop(family, cfg, factory, spec.steps, recipe.hyper(), seed=spec.seed, views_of=tr.views_of)
    finally:
        tr.close()
    if a.out:
        res.save(a.out)
    return 0


def cmd_parity(a, argv) -> int:
    from dataflow_b200.run.driver import Trainer
    from dataflow_b200.run.loop import reference_loop, train_loop
    from dataflow_b200.run.parity import Band, compare
    spec, family, cfg, recipe, factory = _twin_setup(a, argv)
    tr = Trainer(family, cfg, budget_gib=spec.budget_gib, device=spec.device, hyper=recipe.hyper(), seed=spec.seed,
                 kernel_set=spec.kernels, lower_kwargs={"resident_params": True} if spec.resident_params else None)
    try:
        ref = reference_loop(family, cfg, factory, spec.steps, recipe.hyper(), seed=spec.seed, views_of=tr.views_of, log=None)
        eng = train_loop(tr, factory, spec.steps, log=None)
    finally:
        tr.close()
    band = Band.named(a.band or ("fp32" if str(getattr(cfg, "dtype_policy", "")) == "fp32" else "bf16"))
    cmp_ = compare(eng.losses, ref.losses, band)
    for i, (x, y) in enumerate(zip(eng.losses, ref.losses), 1):
        print(f"step {i:4d}  engine {x:.5f}  twin {y:.5f}  rel {abs(x - y) / max(abs(y), 1e-30):.2e}")
    print("PARITY OK" if cmp_ else f"PARITY FAILED at steps {[m[0] for m in cmp_.mismatches]}", f"(worst rel {cmp_.worst_rel:.2e})")
    return 0 if cmp_ else 1


def cmd_smoke(a, argv) -> int:
    from dataflow_b200.run.conductor import run
    from dataflow_b200.run.parity import curves_healthy
    a.steps = a.steps or 6
    a.peak_lr = max(a.peak_lr, 2e-3)
    if a.data is None:
        a.data = "synthetic:vocab=64,mean_len=48,seed=0"          # small id range: learnable in a few steps
    res = run(spec_from_args(a, argv))
    ok = curves_healthy(res.losses)
    print("SMOKE OK" if ok else f"SMOKE FAILED: {res.losses}")
    return 0 if ok else 1


def cmd_scaling(a, argv) -> int:
    import dataclasses
    from dataflow_b200.run.conductor import run
    from dataflow_b200.run.scaling import fit_scaling
    pts, per_gpu = [], 0
    for n in [int(x) for x in str(a.gpu_list).split(",")]:
        spec = dataclasses.replace(spec_from_args(a, argv), world=n)
        res = run(spec)
        skip = min(2, max(len(res.step_wall_s) - 1, 0))
        t = sum(res.step_wall_s[skip:]) / max(len(res.step_wall_s) - skip, 1)
        pts.append((n, res.tokens_per_step / t))
        per_gpu = res.tokens_per_step / n
        print(f"{n} GPU: {pts[-1][1]:,.0f} tok/s")
    fit = fit_scaling(pts, per_gpu)
    print(json.dumps({"points": fit.points, "efficiency": fit.efficiency, "t_compute_ms": fit.t_compute_ms,
                      "t_comm_ms": fit.t_comm_ms}, indent=1))
    return 0


def cmd_peek(a, argv) -> int:
    from dataflow_b200.run.checkpointing import peek, resolve_resume
    print(json.dumps(peek(resolve_resume(a.path)), indent=1, default=str))
    return 0


def cmd_compare(a, argv) -> int:
    from dataflow_b200.run.parity import Band, compare
    x, y = (json.load(open(p))["losses"] for p in (a.a, a.b))
    c = compare(x, y, Band.named(a.band))
    print(f"{'MATCH' if c else 'DIFFER'}: worst rel {c.worst_rel:.3e} at step {c.worst_step}; {len(c.mismatches)} outside band {a.band}")
    return 0 if c else 1


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("train", "reference", "smoke", "parity", "scaling"):
        p = sub.add_parser(name)
        add_run_flags(p)
        if name == "parity":
            p.add_argument("--band", default=None, help="bitwise | fp32 | bf16 | loose")
        if name == "scaling":
            p.add_argument("--gpu-list", default="1,2", help="world sizes to run, comma separated")
    p = sub.add_parser("peek")
    p.add_argument("path")
    p = sub.add_parser("compare")
    p.add_argument("a")
    p.add_argument("b")
    p.add_argument("--band", default="bf16")
    a = ap.parse_args(argv)
    if getattr(a, "opt", None):
        from dataflow_b200.blocks import optim
        known = tuple(optim.OPTIMIZERS) + tuple(optim._PLUGIN_OPTIMIZERS)
        if a.opt not in known:
            ap.error(f"--opt {a.opt}: unknown optimizer (known: {', '.join(known)})")
    # flags that cannot mean anything are refused before a model is built
    for flag, low in (("steps", 0), ("ga_rounds", 1), ("batch", 1), ("max_seq_len", 2), ("gpus", 1), ("fast_budget", 0.0), ("backing_budget", 0.0),
                      ("checkpoint_every", 0), ("warmup_steps", 0)):
        v = getattr(a, flag, None)
        if v is not None and not isinstance(v, str) and v < low:
            ap.error(f"--{flag.replace('_', '-')} {v}: must be at least {low}")
    run = {"train": cmd_train, "reference": cmd_reference, "smoke": cmd_smoke, "parity": cmd_parity,
           "scaling": cmd_scaling, "peek": cmd_peek, "compare": cmd_compare}[a.cmd]
    if os.environ.get("DATAFLOW_TRACEBACK") == "1":
        return run(a, argv)
    from dataflow_b200.sim.policies.pressurefit import PlanningError
    try:
        return run(a, argv)
    except (KeyError, FileNotFoundError, PlanningError) as e:
        # a name that does not exist (preset, optimizer, data scheme, checkpoint) or a budget nothing fits: the user's to fix,
        # one line instead of a traceback (DATAFLOW_TRACEBACK=1 shows where it was raised)
        msg = e.args[0] if isinstance(e, KeyError) and e.args else str(e)
        print(f"train.py {a.cmd}: {msg}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    sys.exit(main())
