#!/usr/bin/env python
"""POSIX double-fork launcher with a pidfile, and its counterpart ``--kill``.

    daemonize.py --pidfile P --logfile L [--cwd D] -- command args...
    daemonize.py --pidfile P --kill            # SIGTERM -> wait -> SIGKILL -> verify the process group is gone

The child is a session leader, so ``--kill`` signals the whole process group by its exact id (never by name).
Role parity: reference ``tools/train/daemonize.py``.
"""
from __future__ import annotations

import argparse
import os
import signal
import sys
import time


def group_alive(pgid: int) -> bool:
    try:
        os.killpg(pgid, 0)
        return True
    except ProcessLookupError:
        return False
    except PermissionError:
        return True


def do_kill(pidfile: str, grace: float = 10.0) -> int:
    try:
        pid = int(open(pidfile).read().strip())
    except (OSError, ValueError):
        print(f"no pidfile {pidfile}", file=sys.stderr)
        return 1
    for sig, wait in ((signal.SIGTERM, grace), (signal.SIGKILL, 5.0)):
        if not group_alive(pid):
            break
        try:
            os.killpg(pid, sig)
        except ProcessLookupError:
            break
        deadline = time.time() + wait
        while time.time() < deadline and group_alive(pid):
            time.sleep(0.05)
    gone = not group_alive(pid)
    if gone:
        try:
            os.unlink(pidfile)
        except OSError:
            pass
    else:
        print(f"process group {pid} survived SIGKILL", file=sys.stderr)
    return 0 if gone else 2


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--pidfile", required=True)
    ap.add_argument("--logfile", default=os.devnull)
    ap.add_argument("--cwd", default=None)
    ap.add_argument("--kill", action="store_true")
    ap.add_argument("command", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    if a.kill:
        return do_kill(a.pidfile)
    cmd = a.command[1:] if a.command and a.command[0] == "--" else a.command
    if not cmd:
        ap.error("no command given")
    if os.fork() > 0:
        return 0                              # the launcher returns at once
    os.setsid()                               # new session: the child leads its own process group
    if os.fork() > 0:
        os._exit(0)
    if a.cwd:
        os.chdir(a.cwd)
    with open(a.pidfile, "w") as f:
        f.write(str(os.getpgrp()))
    log = os.open(a.logfile, os.O_WRONLY | os.O_CREAT | os.O_APPEND, 0o644)
    devnull = os.open(os.devnull, os.O_RDONLY)
    os.dup2(devnull, 0)
    os.dup2(log, 1)
    os.dup2(log, 2)
    os.execvp(cmd[0], cmd)
    return 127


if __name__ == "__main__":
    sys.exit(main())
