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
Multi-GPU (its ZeRO-1 ``zero1rs`` lane through the conductor / fleet loop) is not driven
from here; for N > 1 the arm reports ``unavailable``.
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
        return _unavailable("the reference's multi-GPU lane (conductor + one daemon per GPU, ZeRO-1 over NCCL) is not "
                            "driven by this harness; single-GPU only") if rank == 0 else {}
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
