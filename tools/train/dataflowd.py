#!/usr/bin/env python
"""dataflowd: the engine as a service.

    dataflowd.py start  --socket /tmp/dataflowd.sock --backing-gib 64 --device 0 [--kernels sm100] [--fake]
                        [--peer-name a --peer-listen 0.0.0.0:7000] [--plugin my.module] [--foreground]
    dataflowd.py status --socket PATH
    dataflowd.py stop   --socket PATH

``start`` without ``--foreground`` detaches through ``daemonize.py``.  Role parity: reference
``tools/train/dataflowd.py:27-120``.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def cmd_start(a) -> int:
    if not a.foreground:
        stem = a.socket[:-5] if a.socket.endswith(".sock") else a.socket
        argv = [sys.executable, os.path.join(ROOT, "tools/train/daemonize.py"), "--pidfile", stem + ".pid", "--logfile",
                stem + ".log", "--cwd", ROOT, "--", sys.executable, os.path.abspath(__file__), "start", "--foreground"]
        for k, v in vars(a).items():
            if k in ("cmd", "foreground") or v in (None, False):
                continue
            flag = "--" + k.replace("_", "-")
            if isinstance(v, list):
                for x in v:
                    argv += [flag, str(x)]
            else:
                argv += [flag] if v is True else [flag, str(v)]
        return subprocess.call(argv)
    from dataflow_b200.service import EngineConfig, Server
    cfg = EngineConfig(socket_path=a.socket, slab_backing_gib=a.backing_gib if a.backing_gib == "auto" else float(a.backing_gib),
                       device=None if a.fake or a.device == "cpu" else int(a.device), kernel_set=a.kernels, fake=a.fake,
                       peer_name=a.peer_name, peer_listen=a.peer_listen)
    srv = Server(cfg)
    if not a.no_default_workloads:
        from dataflow_b200.register import register_all
        register_all()                 # the built-in families' resolver kind ("model_family")
    for mod in a.plugin or ():
        __import__(mod)
    srv.serve_forever()
    return 0


def cmd_status(a) -> int:
    from dataflow_b200.service import EngineClient
    try:
        with EngineClient(a.socket, "dataflowd-status", timeout=10.0) as c:
            print(json.dumps({"health": c.health(), "engine": c.engine_status()}, indent=1, default=str))
        return 0
    except (OSError, ConnectionError) as e:
        print(f"no daemon at {a.socket}: {e}", file=sys.stderr)
        return 1


def cmd_stop(a) -> int:
    from dataflow_b200.service import EngineClient
    try:
        with EngineClient(a.socket, "dataflowd-stop", timeout=30.0) as c:
            c.shutdown()
        return 0
    except (OSError, ConnectionError) as e:
        print(f"no daemon at {a.socket}: {e}", file=sys.stderr)
        return 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("start")
    s.add_argument("--socket", default="/tmp/dataflowd.sock")
    s.add_argument("--backing-gib", default="auto")
    s.add_argument("--device", default="0")
    s.add_argument("--kernels", default=None)
    s.add_argument("--fake", action="store_true")
    s.add_argument("--peer-name", default=None)
    s.add_argument("--peer-listen", default=None)
    s.add_argument("--plugin", action="append")
    s.add_argument("--no-default-workloads", action="store_true")
    s.add_argument("--foreground", action="store_true")
    for name in ("status", "stop"):
        p = sub.add_parser(name)
        p.add_argument("--socket", default="/tmp/dataflowd.sock")
    a = ap.parse_args(argv)
    return {"start": cmd_start, "status": cmd_status, "stop": cmd_stop}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
