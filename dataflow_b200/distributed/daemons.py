"""Start, probe and stop ``dataflowd`` daemons on topology hosts (through ``tools/train/daemonize.py``, which
double-forks and records a pidfile), plus the environment every rank gets.
Role parity: reference ``src/dataflow_training/distributed/daemons.py:18-140``.
"""
from __future__ import annotations

import os
import sys
import time
from typing import Mapping

from .hosts import run_on
from .topology import HostSpec, Member

NCCL_DEFAULT_ENV = {"NCCL_DEBUG": "WARN", "TORCH_NCCL_ASYNC_ERROR_HANDLING": "1"}
REPO_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def profiler_command(prefix: str, argv: list[str]) -> list[str]:
    """Wrap ``argv`` so the process records NVTX ranges of tasks and transfers (``DATAFLOW_NVTX=1``); a timeline
    profiler, where one is installed, attaches to these ranges."""
    return ["env", "DATAFLOW_NVTX=1", f"DATAFLOW_TRACE_PREFIX={prefix}", *argv]


TIMELINE_TRACE = "cuda,nvtx,osrt,cublas"


def timeline_profiler(host: HostSpec | None = None) -> str | None:
    """Path of the timeline profiler on this machine (``nsys`` on PATH, or what ``DATAFLOW_NSYS`` names), else None."""
    import shutil
    name = os.environ.get("DATAFLOW_NSYS") or getattr(host, "nsys", None) or "nsys"
    return shutil.which(name)


def timeline_command(profiler: str, out_path: str) -> list[str]:
    """The wrap that records one daemon's timeline between the profiler API's start and stop calls (the conductor sends
    ``profiler_control`` to every daemon around the chosen steps, so the report holds those steps only and the NVTX
    ranges of their tasks and transfers).  ``DATAFLOW_NSYS_EXTRA`` appends capture options without touching this line."""
    argv = [profiler, "profile", f"--trace={TIMELINE_TRACE}", "--capture-range=cudaProfilerApi", "--capture-range-end=stop",
            "-o", out_path, "--force-overwrite", "true"]
    extra = os.environ.get("DATAFLOW_NSYS_EXTRA")
    if extra:
        argv[-4:-4] = extra.split()
    return argv


def daemon_paths(member: Member, root: str = "/tmp", tag: str | None = None) -> dict[str, str]:
    """Runtime files of one daemon.  ``tag`` tells daemons apart that share a host and a device (CPU ranks of one box)."""
    stem = f"{root}/dataflowd.{member.host}.{member.device}" + (f".{tag}" if tag else "")
    return {"socket": stem + ".sock", "pidfile": stem + ".pid", "logfile": stem + ".log"}


def launch(host: HostSpec, member: Member, *, backing_gib: float | str | None = None, kernels: str | None = None,
           fake: bool = False, peer_name: str | None = None, peer_listen: str | None = None, root: str = "/tmp",
           env: Mapping[str, str] | None = None, wait_s: float = 60.0, tag: str | None = None,
           device: str | None = None, wrap: list[str] | None = None) -> dict[str, str]:
    """Start one daemon for ``member`` and wait until its socket answers.  ``device``: what the daemon is told to run on when
    that is not the member's CUDA ordinal (``"cpu"``: the host backend).  ``wrap``: a command prefix that runs INSIDE the
    detached session, around the daemon (``timeline_command(...)``), so a profiler's helpers never hold the launcher open."""
    paths = daemon_paths(member, root, tag)
    repo = host.repo or REPO_ROOT
    py = sys.executable if host.local else host.python
    argv = [py, os.path.join(repo, "tools/train/daemonize.py"), "--pidfile", paths["pidfile"], "--logfile", paths["logfile"],
            "--cwd", repo, "--"]
    for k, v in {**NCCL_DEFAULT_ENV, **dict(env or {})}.items():
        argv += ["env", f"{k}={v}"] if argv[-1] == "--" else [f"{k}={v}"]
    argv += list(wrap or [])
    argv += [py, os.path.join(repo, "tools/train/dataflowd.py"), "start", "--foreground", "--socket", paths["socket"],
             "--backing-gib", str(backing_gib if backing_gib is not None else host.backing_gib)]
    argv += ["--fake"] if fake else ["--device", str(device if device is not None else member.device)]
    if kernels:
        argv += ["--kernels", kernels]
    if peer_name:
        argv += ["--peer-name", peer_name]
    if peer_listen:
        argv += ["--peer-listen", peer_listen]
    run_on(host, argv, timeout=wait_s)
    deadline = time.time() + wait_s
    while time.time() < deadline:
        if alive(host, member, root, tag):
            return paths
        time.sleep(0.2)
    raise TimeoutError(f"daemon for {member.key} did not come up within {wait_s:.0f} s (log: {paths['logfile']})")


def alive(host: HostSpec, member: Member, root: str = "/tmp", tag: str | None = None) -> bool:
    paths = daemon_paths(member, root, tag)
    py = sys.executable if host.local else host.python
    repo = host.repo or REPO_ROOT
    r = run_on(host, [py, os.path.join(repo, "tools/train/dataflowd.py"), "status", "--socket", paths["socket"]],
               check=False, timeout=30)
    return r.returncode == 0


def wait_exit(host: HostSpec, member: Member, root: str = "/tmp", timeout: float = 60.0, tag: str | None = None) -> bool:
    deadline = time.time() + timeout
    while time.time() < deadline:
        if not alive(host, member, root, tag):
            return True
        time.sleep(0.2)
    return False


def kill(host: HostSpec, member: Member, root: str = "/tmp", tag: str | None = None) -> None:
    """Stop by pidfile: signal, wait, escalate, verify the process group is gone (``daemonize.py --kill``)."""
    paths = daemon_paths(member, root, tag)
    py = sys.executable if host.local else host.python
    repo = host.repo or REPO_ROOT
    run_on(host, [py, os.path.join(repo, "tools/train/daemonize.py"), "--pidfile", paths["pidfile"], "--kill"], check=False,
           timeout=60)
