"""Reference arm of the benchmark: runs the UNMODIFIED reference (installed under
``baseline/_ref``) through its own public API and stock code path — its preset
(``resolve_preset``), its planner (``plan_at_budget``), its in-process daemon
(``engine_client``), its kernels and its step loop (``run_engine``) — on the same
metric and configuration as our arm, and prints the same JSON line with
``"impl": "reference"``.

What the reference can run of the configuration: its ``llama3_8b`` preset at seq 4096,
131072 tokens per step, AdamW with its all-bf16 state policy (it has no fp32-master
lane), one GPU per daemon.  It has no B200 hardware preset and raises on an unknown device;
the harness adds a ``b200`` row to its ``HW_PRESETS`` table at run time (the route its own
error message names) and touches none of its files.
Multi-GPU: rank 0 of the launch acts as the reference's conductor — its ``run/conductor.run`` starts one ``dataflowd`` per GPU
(the reference's own ``tools/train/{daemonize,dataflowd}.py``, copied beside the installed packages together with its
``pyproject.toml`` because the conductor looks them up under the repository root), links them, creates the NCCL peer group and
runs its lock-step fleet loop with data parallelism over its ``zero1rs`` optimizer sharding, the same rounds per GPU as at
N = 1 (weak scaling).  The other ranks of the launch have nothing to do and exit.
"""
from __future__ import annotations

import json
import os
import sys
import time
from dataclasses import replace


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}


def run_reference_arm(a) -> dict:
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    here = os.path.dirname(os.path.abspath(__file__))
    ref = os.path.join(here, "_ref")
    if not os.path.isdir(os.path.join(ref, "dataflow_training")):
        return _unavailable("baseline/_ref is not installed on this machine") if rank == 0 else {}
    if world > 1 or a.gpus > 1:
        return _run_fleet(a, max(world, a.gpus), here, ref) if rank == 0 else {}
    sys.path.insert(0, ref)
    try:
        import torch
        from dataflow_training.run import presets as P
        from dataflow_training.run.driver import engine_client, plan_at_budget, run_engine
        from dataflow_training.run.recipe import Recipe
        from dataflow_training.data.pipeline import pipeline_from_args
    except Exception as e:       # noqa: BLE001
        return _unavailable(f"reference import failed: {type(e).__name__}: {e}")
    try:
        base = P.resolve_preset(a.preset)
        rounds = max(a.tokens_per_gpu // (a.seq_len * a.batch), 1)
        cfg = replace(base, seq_len=a.seq_len, batch=a.batch, grad_accum_rounds=rounds)
        budget = a.budget_gib if a.budget_gib is not None else 60.0
        steps = a.warmup + a.steps
        recipe = Recipe(peak_lr=3e-4, min_lr=3e-5, warmup_steps=max(1, steps // 3), total_steps=steps)
        tokens_step = cfg.max_tokens * cfg.grad_accum_rounds
        # synthetic uniform ids, full windows of seq_len (mean_len large and trimmed to the window)
        spec = f"synthetic:mean_len={8 * a.seq_len},seed=0,long_policy=trim"
        logs: list[str] = []

        factory = pipeline_from_args(cfg, spec)      # a DataPipeline is itself the factory run_engine calls with a cursor

        t_plan = time.perf_counter()
        # The reference has no B200 row in its HW_PRESETS table, and its stock path (planning AND the
        # init task inside the daemon) calls resolve_hardware(), which raises on an unknown device with
        # "add one to HW_PRESETS or pass hw=...".  The harness takes the first route its message names:
        # it adds a row to that module-level table at run time (measured peaks of this pool's B200); no
        # file of the reference is touched.
        from dataflow_training.lowering import shaped_program as ref_sp
        ref_sp.HW_PRESETS.setdefault("b200", dict(peak_bf16_tflops=1669.0, matmul_eff=0.75, attn_eff=0.45,
                                                  mem_bw_gbs=6524.0, mem_eff=0.8, pcie_gbs=52.0))
        # The reference's own training entry prices the tasks by profiling them on the device before it plans
        # (run/loop.py -> run/profiling.py load_or_profile); the arm does the same unless DFB_REF_COSTS=roofline asks for
        # the hardware-row estimate.  If the profiling pass fails on this device the arm falls back to the estimate and
        # says so in ``plan.costs``.
        costs = "measured" if os.environ.get("DFB_REF_COSTS", "measured") != "roofline" else "roofline"
        planned = None
        if costs == "measured":
            try:
                planned = plan_at_budget(replace(cfg, num_steps=1), budget, measured=True, backing_gib=150.0)
            except Exception as e:       # noqa: BLE001
                costs = f"roofline (measured profiling failed: {type(e).__name__}: {str(e)[:120]})"
        if planned is None:
            planned = plan_at_budget(replace(cfg, num_steps=1), budget, measured=False, backing_gib=150.0)
        plan_s = time.perf_counter() - t_plan
        stamps: list[float] = []

        def on_log(*x, **k):
            line = " ".join(map(str, x))
            logs.append(line)
            if "] step " in line and "tok/s" in line:
                stamps.append(time.perf_counter())        # one line per step (log_every=1), printed right after the step's run

        with engine_client(backing_gib=150.0, log=lambda *x, **k: None) as client:
            res = run_engine(client, cfg, recipe, factory, steps, budget_gib=budget, seed=11, planned=planned,
                             log=on_log, log_every=1)
        tail = res.step_wall_s[a.warmup:] or res.step_wall_s
        s_per_step = sum(tail) / len(tail)
        value = tokens_step / s_per_step
        # End to end: the whole loop iteration of the reference's step loop — staging the step's tokens and targets into
        # the daemon's pinned store (put_object), the run (whose first transfers copy them to the device) and the loss
        # fetch — taken from the time between consecutive per-step log lines.
        e2e = None
        if len(stamps) == steps and steps - a.warmup >= 1 and a.warmup >= 1:
            span = stamps[-1] - stamps[a.warmup - 1]
            e2e = {"value": tokens_step * (steps - a.warmup) / span, "unit": "tokens/s",
                   "h2d_bytes_per_step": 2 * 4 * tokens_step, "d2h_bytes_per_step": 4 * cfg.grad_accum_rounds,
                   "how": "wall clock between the reference's per-step log lines: put_object of the step's ids into its "
                          "pinned store + run + loss fetch"}
        return {
            "metric": "train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": len(tail),
            "warmup": a.warmup, "ms_per_step": s_per_step * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / 12618.0, "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": {"model": a.preset, "global_batch": tokens_step // a.seq_len, "seq_len": a.seq_len,
                       "tokens_per_step": tokens_step, "parallelism": "solo", "fast_budget_gib": budget,
                       "dtype_policy": "all-bf16 (the reference has no fp32-master lane)", "optimizer": "adamw",
                       "hw_preset": "b200 row added to the reference's HW_PRESETS table at run time",
                       "timing": "reference's own per-step wall clock (its step loop blocks on the loss fetch)"},
            "plan": {"predicted_ms_per_step": planned.makespan_us / 1e3, "plan_s": plan_s, "costs": costs},
            "e2e": e2e,
            "loss": res.losses[-1] if res.losses else None,
            "gpu_launches": None, "torch": torch.__version__,
        }
    except Exception as e:       # noqa: BLE001
        import traceback
        tb = traceback.format_exc().strip().splitlines()
        dump = os.environ.get("DFB_REF_TRACEBACK")
        if dump:
            with open(dump, "w") as f:
                f.write("\n".join(tb) + "\n\n" + "\n".join(logs if "logs" in dir() else []))
        return _unavailable(f"reference run failed: {type(e).__name__}: {e} | {tb[-3] if len(tb) > 2 else ''}")


def _host_backing_gib(n: int) -> float:
    """Pinned host store per daemon: the reference's 150 GiB default where the box has it, else an equal share of 60 % of the
    memory that is free now (the planner is told the capacity and plans within it)."""
    avail = None
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    avail = int(line.split()[1]) * 1024
    except OSError:
        pass
    for p in ("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory/memory.limit_in_bytes"):
        try:
            v = open(p).read().strip()
            if v.isdigit() and int(v) < (1 << 60):
                avail = min(avail, int(v)) if avail else int(v)
        except OSError:
            pass
    if not avail:
        return 64.0
    return max(min(150.0, 0.6 * avail / n / 2 ** 30), 8.0)


def _ensure_git(ref: str) -> None:
    """The reference's conductor refuses to start a fleet unless ``git rev-parse HEAD`` answers at its repository root (its
    mixed-version guard).  The installed tree is no checkout, so it gets an empty history of its own; no file changes."""
    import subprocess
    if os.path.isdir(os.path.join(ref, ".git")):
        return
    env = dict(os.environ, GIT_AUTHOR_NAME="bench", GIT_AUTHOR_EMAIL="bench@localhost", GIT_COMMITTER_NAME="bench",
               GIT_COMMITTER_EMAIL="bench@localhost")
    for cmd in (["git", "init", "-q"], ["git", "add", "-A"], ["git", "commit", "-q", "-m", "installed reference"]):
        subprocess.run(cmd, cwd=ref, env=env, check=True, capture_output=True)


def _run_fleet(a, world: int, here: str, ref: str) -> dict:
    import socket
    import tempfile
    for need in ("tools/train/dataflowd.py", "tools/train/daemonize.py", "pyproject.toml"):
        if not os.path.exists(os.path.join(ref, need)):
            return _unavailable(f"baseline/_ref/{need} is missing: copy the reference's tools/ and pyproject.toml beside the "
                                f"installed packages")
    sys.path.insert(0, ref)
    os.environ["PYTHONPATH"] = ref + os.pathsep + os.environ.get("PYTHONPATH", "")
    os.environ.pop("OMP_NUM_THREADS", None)       # the launcher's one-thread default would also bind the daemons it never sees
    logs: list[str] = []
    cwd = os.getcwd()
    try:
        import torch
        from dataflow_training.data.pipeline import pipeline_from_args
        from dataflow_training.distributed.parallelism import ParallelismScheme
        from dataflow_training.distributed.topology import GroupSpec, HostSpec, Topology
        from dataflow_training.lowering import shaped_program as ref_sp
        from dataflow_training.run import presets as P
        from dataflow_training.run.conductor import run as conductor_run
        from dataflow_training.run.recipe import Recipe
    except Exception as e:       # noqa: BLE001
        return _unavailable(f"reference import failed: {type(e).__name__}: {e}")
    try:
        if torch.cuda.device_count() < world:
            return _unavailable(f"{world} GPUs asked, {torch.cuda.device_count()} visible")
        sys.path.insert(0, here)
        from ref_launch import B200_ROW
        _ensure_git(ref)
        ref_sp.HW_PRESETS.setdefault("b200", dict(B200_ROW))          # the conductor prices tasks in this process
        base = P.resolve_preset(a.preset)
        per_rank = max(a.tokens_per_gpu // (a.seq_len * a.batch), 1)
        cfg = replace(base, seq_len=a.seq_len, batch=a.batch, grad_accum_rounds=per_rank * world)
        budget = a.budget_gib if a.budget_gib is not None else 60.0
        steps = a.warmup + a.steps
        recipe = Recipe(peak_lr=3e-4, min_lr=3e-5, warmup_steps=max(1, steps // 3), total_steps=steps)
        tokens_step = cfg.max_tokens * cfg.grad_accum_rounds
        feed = pipeline_from_args(cfg, f"synthetic:mean_len={8 * a.seq_len},seed=0,long_policy=trim")
        backing = _host_backing_gib(world)
        # One GPU per daemon through CUDA_VISIBLE_DEVICES (device 0 inside each): the reference's NCCL bring-up thread never
        # selects a device, so on a box where every daemon sees every GPU all ranks would open the communicator on GPU 0.
        visible = [v for v in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if v] or [str(i) for i in range(world)]

        def interpreter(i):
            return f"env CUDA_VISIBLE_DEVICES={visible[i]} {sys.executable} {os.path.join(here, 'ref_launch.py')}"

        def free_port():
            with socket.socket() as s:
                s.bind(("127.0.0.1", 0))
                return s.getsockname()[1]

        names = [f"gpu{i}" for i in range(world)]
        hosts = {n: HostSpec(name=n, peer_listen=f"127.0.0.1:{free_port()}", ssh=None, python=interpreter(i), repo=ref,
                             backing_gib=backing, budget_gib=budget, device=0) for i, n in enumerate(names)}
        topo = Topology(conductor=names[0], hosts=hosts,
                        groups={"dp": GroupSpec(name="dp", members=tuple(names), backend="nccl")}, source="<bench: one box>")
        scheme = ParallelismScheme.data_parallel((per_rank,) * world, responsibility="zero1rs")
        stamps: list[float] = []

        def on_log(*x, **k):
            line = " ".join(map(str, x))
            logs.append(line)
            if "[fleet] step " in line and "tok/s" in line:
                stamps.append(time.perf_counter())

        work = tempfile.mkdtemp(prefix="dfb_ref_fleet_")
        os.chdir(work)                 # the reference writes its profile cache and run files relative to the cwd
        t0 = time.perf_counter()
        res = conductor_run(cfg, recipe, feed, steps, scheme=scheme, budgets=(budget,) * world, backing=(backing,) * world,
                            topology=topo, group="dp", seed=11, log=on_log, log_every=1, warm_profiles=True,
                            prof_dir=os.path.join(work, "prof"))
        total_s = time.perf_counter() - t0
        tail = res.step_wall_s[a.warmup:] or res.step_wall_s
        s_per_step = sum(tail) / len(tail)
        value = tokens_step / s_per_step
        e2e = None
        if len(stamps) == steps and steps - a.warmup >= 1 and a.warmup >= 1:
            span = stamps[-1] - stamps[a.warmup - 1]
            e2e = {"value": tokens_step * (steps - a.warmup) / span, "unit": "tokens/s", "h2d_bytes_per_step": 2 * 4 * tokens_step,
                   "d2h_bytes_per_step": 4 * cfg.grad_accum_rounds,
                   "how": "wall clock between the conductor's per-step log lines: put_object of every rank's ids into its daemon's "
                          "pinned store + the lock-step runs + loss fetches"}
        return {
            "metric": "train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": len(tail),
            "warmup": a.warmup, "ms_per_step": s_per_step * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / 12618.0, "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": {"model": a.preset, "global_batch": tokens_step // a.seq_len, "seq_len": a.seq_len, "tokens_per_step": tokens_step,
                       "parallelism": f"dp{world} zero1rs over NCCL, one dataflowd per GPU", "fast_budget_gib": budget,
                       "host_backing_gib_per_rank": backing,
                       "dtype_policy": "all-bf16 (the reference has no fp32-master lane)", "optimizer": "adamw",
                       "hw_preset": "b200 row added to the reference's HW_PRESETS table at run time (conductor and daemons)",
                       "timing": "the conductor's own per-step wall clock (upload + lock-step runs + loss fetch)"},
            "plan": {"costs": "measured (its --warm-profiles stage)", "total_s": total_s},
            "e2e": e2e, "loss": res.losses[-1] if res.losses else None, "gpu_launches": None, "torch": torch.__version__,
        }
    except Exception as e:       # noqa: BLE001
        import traceback
        tb = traceback.format_exc().strip().splitlines()
        dump = os.environ.get("DFB_REF_TRACEBACK")
        if dump:
            os.chdir(cwd)
            with open(dump, "w") as f:
                f.write("\n".join(tb) + "\n\n" + "\n".join(logs))
        return _unavailable(f"reference fleet run failed: {type(e).__name__}: {e} | {tb[-3] if len(tb) > 2 else ''}")
    finally:
        os.chdir(cwd)
