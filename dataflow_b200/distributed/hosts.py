"""Run things on a host of the topology: locally, or through ssh for hosts with an address; forward a remote
daemon's unix socket to a local path; fetch a file.  Role parity: reference
``src/dataflow_training/distributed/hosts.py:32-110``.
"""
from __future__ import annotations

import shlex
import shutil
import subprocess
from typing import Sequence

from .topology import HostSpec

SSH_OPTS = ["-o", "BatchMode=yes", "-o", "StrictHostKeyChecking=accept-new", "-o", "ConnectTimeout=10"]


def command_for(host: HostSpec, argv: Sequence[str], cwd: str | None = None) -> list[str]:
    """The argv that runs ``argv`` on ``host`` (unchanged for the local machine)."""
    if host.local:
        return list(argv)
    inner = " ".join(shlex.quote(a) for a in argv)
    if cwd or host.repo:
        inner = f"cd {shlex.quote(cwd or host.repo)} && {inner}"
    return ["ssh", *SSH_OPTS, host.address, inner]


def run_on(host: HostSpec, argv: Sequence[str], *, cwd: str | None = None, timeout: float | None = None,
           check: bool = True, capture: bool = True) -> subprocess.CompletedProcess:
    cmd = command_for(host, argv, cwd)
    return subprocess.run(cmd, cwd=cwd if host.local else None, timeout=timeout, check=check,
                          capture_output=capture, text=True)


def uds_forward(host: HostSpec, remote_socket: str, local_socket: str) -> subprocess.Popen | None:
    """``ssh -N -L local:remote`` for a remote daemon's unix socket; ``None`` for the local machine."""
    if host.local:
        return None
    return subprocess.Popen(["ssh", *SSH_OPTS, "-N", "-L", f"{local_socket}:{remote_socket}", host.address])


def fetch_file(host: HostSpec, remote_path: str, local_path: str) -> None:
    if host.local:
        shutil.copyfile(remote_path, local_path)
        return
    subprocess.run(["scp", *SSH_OPTS, f"{host.address}:{remote_path}", local_path], check=True)
