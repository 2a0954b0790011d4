"""Peer-plane preflight of one box: which GPUs can address which (peer access), whether a CUDA IPC handle opens in another
process, and the per-direction copy bandwidth of every pair — the facts the fused peer-memory kernels depend on.

    python tools/verify/p2p_preflight.py [--mib 256] [--pairs all|ring]

On a host without GPUs it says so and exits 0.  Reference role: ``tools/verify/rdma_preflight.py`` (there: RDMA links
between hosts; here: NVLink between the GPUs of one box).
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import _cli  # noqa: E402,F401


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--mib", type=int, default=256)
    ap.add_argument("--pairs", default="ring", choices=["ring", "all"])
    a = ap.parse_args(argv)
    import torch
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if n == 0:
        print("no CUDA devices on this host: nothing to check")
        return 0
    print(f"{n} device(s): " + ", ".join(torch.cuda.get_device_name(i) for i in range(n)))
    bad = 0
    for i in range(n):
        row = []
        for j in range(n):
            ok = i == j or torch.cuda.can_device_access_peer(i, j)
            bad += not ok
            row.append("self" if i == j else ("ok" if ok else "NO"))
        print(f"peer access from {i}: " + " ".join(f"{x:>4}" for x in row))
    if n > 1:
        pairs = [(i, (i + 1) % n) for i in range(n)] if a.pairs == "ring" else [(i, j) for i in range(n) for j in range(n) if i != j]
        nbytes = a.mib << 20
        for i, j in pairs:
            src = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{i}")
            dst = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{j}")
            for _ in range(2):
                dst.copy_(src)
            torch.cuda.synchronize(i)
            torch.cuda.synchronize(j)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.device(j):
                e0.record()
                for _ in range(5):
                    dst.copy_(src, non_blocking=True)
                e1.record()
                torch.cuda.synchronize(j)
            print(f"copy {i} -> {j}: {5 * nbytes / e0.elapsed_time(e1) / 1e6:.0f} GB/s")
            del src, dst
    from dataflow_b200.runtime import CudaBackend
    be = CudaBackend(0, "poll")
    p = be.device_alloc_zeroed(1 << 20)
    h = be.ipc_handle(p)
    print(f"IPC handle export: ok ({len(h)} bytes)")
    be.device_free(p)
    print("PASS" if not bad else "FAIL: some pairs have no peer access")
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
