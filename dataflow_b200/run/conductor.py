"""``run(...)``: from a run specification to a finished ``RunResult``.

World size 1 runs in this process.  Larger worlds launch one process per GPU on this node through
``torch.distributed.run`` (rendezvous on 127.0.0.1) with ``dataflow_b200.run.rank_main`` as the entry; rank 0
writes the result file this function returns.  A run that checkpoints takes an exclusive ``flock`` on its
checkpoint directory for its whole lifetime, so two runs can never interleave step directories.
Role parity: reference ``src/dataflow_training/run/conductor.py:146-452`` (there: daemons + a conductor; here the
ranks are the processes themselves).
"""
from __future__ import annotations

import dataclasses
import fcntl
import json
import os
import socket
import subprocess
import sys
import tempfile
from typing import Any, Mapping

from .driver import RunResult


@dataclasses.dataclass
class RunSpec:
    preset: str
    steps: int
    overrides: dict[str, Any] = dataclasses.field(default_factory=dict)        # config fields (seq_len, batch, ...)
    recipe: dict[str, Any] = dataclasses.field(default_factory=dict)
    data: str | None = None
    packing_policy: str = "ffd"
    allow_round_split: bool = False
    capture: str | None = None
    budget_gib: float | None = None
    device: int | None = 0                  # None = CPU backend
    world: int = 1
    parallel: str = "fsdp"                  # fsdp | zero3 | zero1 | co | tp | ep (world > 1)
    tp_size: int | None = None              # with ``tp``: ranks per tensor-parallel group; the job is a (world / tp_size) x tp_size mesh
    ep_size: int | None = None              # with ``ep``: ranks per expert-parallel group; the groups are replicas of each other
    rounds: list[int] | None = None         # weighted data parallelism (with ``co``): rounds each rank runs per step
    seed: int = 0
    profile: bool = False
    recompute: bool = True
    kernels: str | None = None
    resident_params: bool = True
    checkpoint_every: int = 0
    checkpoint_dir: str | None = None
    checkpoint_keep_last: int | None = None
    checkpoint_redundancy: int | None = None   # ranks that write their copy of replicated objects (default: all)
    resume: str | None = None
    max_restarts: int = 0                   # relaunch a failed multi-rank job from its newest complete checkpoint, this many times
    out: str | None = None
    devices: list[int] | None = None        # CUDA ordinal of every rank (from a topology group); default: rank r on device r
    backend: str = "auto"                   # auto | peer (kernels over peer memory) | nccl (library collectives around library ops)
    backing_budget_gib: float | None = None # refuse the run when its pinned host store would exceed this
    prof_dir: str | None = None             # per-step engine traces of the steps in the window land here
    profile_start_before_step: int = 0      # 1-indexed; 0 = no window
    profile_stop_after_step: int = 0
    launcher: str = "process"               # process: one rank per process under torch.distributed.run; fleet: one dataflowd per rank (run/fleet.py)
    warm_profiles: bool = False             # measure and cache the task costs, then stop
    refresh_profiles: bool = False          # ignore cached task costs
    argv: list[str] = dataclasses.field(default_factory=list)

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self))

    @staticmethod
    def from_json(s: str) -> "RunSpec":
        return RunSpec(**json.loads(s))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class RunLock:
    def __init__(self, directory: str | None):
        self.path = os.path.join(directory, ".run.lock") if directory else None
        self.f = None

    def __enter__(self):
        if self.path:
            os.makedirs(os.path.dirname(self.path), exist_ok=True)
            self.f = open(self.path, "w")
            try:
                fcntl.flock(self.f, fcntl.LOCK_EX | fcntl.LOCK_NB)
            except BlockingIOError:
                self.f.close()
                raise RuntimeError(f"another run holds {self.path}: two runs must not share a checkpoint directory") from None
            self.f.write(str(os.getpid()))
            self.f.flush()
        return self

    def __exit__(self, *exc):
        if self.f:
            fcntl.flock(self.f, fcntl.LOCK_UN)
            self.f.close()


def _failure_markers(out: str) -> list[str]:
    import glob
    return sorted(glob.glob(glob.escape(out) + ".failure.rank*"))


def _read_failure_kinds(out: str) -> list[tuple[str, str]]:
    kinds = []
    for path in _failure_markers(out):
        try:
            d = json.loads(open(path).read())
            kinds.append((str(d.get("kind", "host")), str(d.get("message", ""))))
        except (OSError, ValueError):
            kinds.append(("host", "unreadable failure marker"))
    return kinds


def run(spec: RunSpec, log=print) -> RunResult:
    if spec.launcher == "fleet":
        from .fleet import run_fleet
        return run_fleet(spec, log=log)
    if spec.launcher != "process":
        raise ValueError(f"--launcher is process or fleet, not {spec.launcher!r}")
    with RunLock(spec.checkpoint_dir if spec.checkpoint_every else None):
        if spec.world <= 1:
            from .rank_main import run_rank
            return run_rank(spec, log=log)
        out = spec.out or os.path.join(tempfile.mkdtemp(prefix="dataflow_run_"), "result.json")
        spec = dataclasses.replace(spec, out=out)
        env = dict(os.environ)
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
        attempt = 0
        while True:
            # a fresh port per attempt: the previous rendezvous may still hold its own
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={spec.world}",
                   "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
                   "-m", "dataflow_b200.run.rank_main", "--spec", spec.to_json()]
            for stale in _failure_markers(out):
                os.unlink(stale)
            proc = subprocess.run(cmd, env=env)
            if proc.returncode == 0:
                break
            # a rank that failed in Python says what kind of failure it was; only host-side failures (an exception, a rank
            # that left, a peer that timed out) are worth a relaunch — a device error would be re-run unchanged
            kinds = _read_failure_kinds(out)
            device = [m for k, m in kinds if k == "device"]
            if device:
                raise RuntimeError(f"the {spec.world}-rank job stopped on a device error and is not restarted: {device[0]}")
            from .checkpointing import resolve_resume
            newest = resolve_resume("latest", spec.checkpoint_dir) if spec.checkpoint_dir else None
            if attempt >= int(spec.max_restarts) or not newest:
                raise RuntimeError(f"the {spec.world}-rank job exited with code {proc.returncode}"
                                   + (f" after {attempt} restart(s)" if attempt else ""))
            attempt += 1
            log(f"the job exited with code {proc.returncode}: restart {attempt} of {spec.max_restarts} from {newest}")
            spec = dataclasses.replace(spec, resume=newest)
        d = json.loads(open(out).read())
        d["meta"]["restarts"] = attempt
        if attempt:
            with open(out, "w") as f:                   # the result file says how the job got to its end
                json.dump(d, f)
        return RunResult(d["losses"], d["step_wall_s"], d["tokens_per_step"], d["meta"])
