"""Measured task costs.  Every distinct task *signature* of a program is timed on the
real device by running a one-layer, two-round cut of the same model through the
engine (so inputs are real activations, not zeros: zero inputs under-price dense
kernels because the chip clocks higher on them) and reading the per-task intervals
of a warm step; the result is cached on disk keyed by geometry, kernel set, device
and library versions.  Role parity: reference ``src/dataflow_training/run/profiling.py:78-964``.
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
import os
from pathlib import Path
from typing import Any, Mapping

from ..core import Program, TaskSpec

PROFILE_CACHE_REV = 5


def task_signature(t: TaskSpec) -> str:
    acc = "acc" if any(m.startswith("dW") for m in t.mutates) else "new"
    lvl = int(t.block_params.get("recompute_level", 0)) if t.block_params else 0
    return f"{t.compute_block_key}|{acc}|l{lvl}"


def apply_measured_costs(program: Program, measured: Mapping[str, float] | None) -> Program:
    if not measured:
        return program
    tasks = []
    for t in program.tasks:
        us = measured.get(task_signature(t))
        tasks.append(dataclasses.replace(t, runtime_us=float(us)) if us else t)
    md = dict(program.metadata)
    md["costs"] = "measured"
    return dataclasses.replace(program, tasks=tuple(tasks), metadata=md)


def _cache_path(key: str) -> Path:
    root = Path(os.environ.get("DATAFLOW_PROFILE_CACHE", Path.home() / ".cache" / "dataflow_b200" / "profiles"))
    root.mkdir(parents=True, exist_ok=True)
    return root / f"{key}.json"


def _ops_build_id() -> str:
    """Digest of the compiled kernel library (and the GEMM path override): new kernels, new measurements."""
    import glob
    h = hashlib.sha256(os.environ.get("DFB_GEMM_PATH", "").encode())
    for f in sorted(glob.glob(str(Path(__file__).resolve().parent.parent / "ops" / "_ops*.so"))):
        with open(f, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def profile_key(trainer, cfg) -> str:
    import torch
    desc = {"rev": PROFILE_CACHE_REV, "cfg": {k: (v if isinstance(v, (int, float, str, bool, type(None))) else str(v))
                                              for k, v in dataclasses.asdict(cfg).items() if k not in ("n_layers", "grad_accum_rounds", "name")},
            "kernels": trainer.K.describe(), "kernel_build": _ops_build_id(), "torch": torch.__version__,
            "device": torch.cuda.get_device_name(trainer.device) if trainer.device is not None else "cpu"}
    return hashlib.sha256(json.dumps(desc, sort_keys=True).encode()).hexdigest()[:20]


class PcieContender:
    """Keeps both PCIe directions busy with pinned copies on two side streams while tasks are timed: in a real step the plan's
    offloads and prefetches run beside the kernels and take memory bandwidth from them, so costs measured on an idle bus are
    optimistic.  Off by default (``DATAFLOW_PROFILE_CONTENDER=1``); a no-op without a device."""

    def __init__(self, device: int | None, mib: int = 256):
        self.device, self.mib = device, int(mib)
        self._stop = None
        self._thread = None
        self.copies = 0

    def __enter__(self):
        if self.device is None:
            return self
        import threading
        import torch
        self._stop = threading.Event()
        n = self.mib << 20
        host_a, host_b = torch.empty(n, dtype=torch.uint8).pin_memory(), torch.empty(n, dtype=torch.uint8).pin_memory()
        dev = torch.device("cuda", self.device)
        dev_a, dev_b = torch.empty(n, dtype=torch.uint8, device=dev), torch.empty(n, dtype=torch.uint8, device=dev)
        up, down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

        def loop():
            while not self._stop.is_set():
                with torch.cuda.stream(up):
                    dev_a.copy_(host_a, non_blocking=True)
                with torch.cuda.stream(down):
                    host_b.copy_(dev_b, non_blocking=True)
                up.synchronize()
                down.synchronize()
                self.copies += 2
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        if self._stop is not None:
            self._stop.set()
            self._thread.join(timeout=30)
        return False


def profile_program(trainer, program: Program | None = None, *, steps: int = 3, use_cache: bool = True,
                    soak_seconds: float | None = None, contender: bool | None = None) -> dict[str, float]:
    """signature → median measured µs, from a 1-layer 2-round cut of ``trainer.cfg`` on ``trainer.device``.
    ``soak_seconds`` (``DATAFLOW_PROFILE_SOAK``): keep stepping each cut until that much time has passed before the ``steps``
    steps that count — a power-capped device settles at lower clocks than its first burst shows.  ``contender``
    (``DATAFLOW_PROFILE_CONTENDER=1``): time the tasks beside busy PCIe lanes (``PcieContender``)."""
    import time
    from .driver import Trainer, synthetic_rounds
    cfg = trainer.cfg
    soak = float(os.environ.get("DATAFLOW_PROFILE_SOAK", 0.0)) if soak_seconds is None else float(soak_seconds)
    contend = (os.environ.get("DATAFLOW_PROFILE_CONTENDER") == "1") if contender is None else bool(contender)
    key = profile_key(trainer, cfg) + (f"-soak{soak:g}" if soak else "") + ("-contended" if contend else "")
    path = _cache_path(key)
    if use_cache and path.exists() and os.environ.get("DATAFLOW_PROFILE_REFRESH") != "1":
        return json.loads(path.read_text())
    out: dict[str, list[float]] = {}
    for levels in (None, {0: 1}, {0: 2}):
        small = dataclasses.replace(cfg, n_layers=1, grad_accum_rounds=2)
        tr = Trainer(trainer.fam.name, small, budget_gib=None, device=trainer.device, hyper=trainer.hyper,
                     kernels=trainer.K, recompute=False, profile=False,
                     lower_kwargs={"recompute_levels": levels} if levels else None)
        try:
            with PcieContender(trainer.device if contend else None):
                t0, s = time.perf_counter(), 0
                while soak and time.perf_counter() - t0 < soak:          # settle the clocks; these steps are not sampled
                    tr.step(synthetic_rounds(small, tr.rounds, tr.T, getattr(small, "vocab_size"), 7, s))
                    s += 1
                by_id = {t.id: t for t in tr.program.tasks}
                for k in range(steps):
                    tr.step(synthetic_rounds(small, tr.rounds, tr.T, getattr(small, "vocab_size"), 7, s + k))
                    if k == 0 and not soak:
                        continue                                          # the first step of a cold cut warms kernels and pools
                    for iv in tr.last_result.trace.by_track("compute"):
                        t = by_id.get(iv.name)
                        if t is not None:
                            out.setdefault(task_signature(t), []).append(iv.end_us - iv.start_us)
        finally:
            tr.close()
    med = {k: sorted(v)[len(v) // 2] for k, v in out.items()}
    if use_cache:
        path.write_text(json.dumps(med, indent=1))
    return med


class ProfileWindow:
    """Steps ``start .. stop`` (1-indexed, inclusive) of a run under observation: the CUDA profiler API is switched on before
    step ``start`` and off after step ``stop`` (an external profiler attached with capture-range = profiler API sees exactly
    those steps), and each step's engine trace — every task and copy with its start and end — is written beside a summary
    to ``<dir>/step_<n>.rank<r>.json``.  Reference role: ``--profile-start-before-step`` / ``--profile-stop-after-step`` /
    ``--prof-dir`` of ``tools/train/train.py:408-457``."""

    def __init__(self, directory: str | None, start: int, stop: int, rank: int = 0):
        self.dir, self.start, self.stop, self.rank = directory, int(start), int(stop or start), int(rank)
        self.active = False
        self.written: list[str] = []

    def __bool__(self):
        return self.start > 0

    def before(self, step: int, trainer) -> None:
        if step == self.start and not self.active:
            self.active = True
            if trainer.device is not None:
                import torch
                torch.cuda.synchronize()
                torch.cuda.profiler.start()

    def after(self, step: int, trainer) -> None:
        if not self.active:
            return
        if self.dir:
            from ..runtime import trace_to_dict
            from .trace_report import summarize_trace
            os.makedirs(self.dir, exist_ok=True)
            res = trainer.last_result
            path = os.path.join(self.dir, f"step_{step:06d}.rank{self.rank}.json")
            with open(path, "w") as f:
                json.dump({"step": step, "rank": self.rank, "predicted_makespan_us": trainer.planned.makespan_us,
                           "measured_makespan_us": res.makespan_us, "summary": summarize_trace(trainer.program, res),
                           "trace": trace_to_dict(res.trace)}, f)
            self.written.append(path)
        if step >= self.stop:
            self.active = False
            if trainer.device is not None:
                import torch
                torch.cuda.synchronize()
                torch.cuda.profiler.stop()
