"""Boot-time bandwidth probe of the daemon's host side: what its own slab delivers for a host copy, a bf16 add (the host
half of a gradient reduction on the host-memory lane) and, on a device, the two PCIe directions.  The figures land in
``engine_status`` so a conductor can see a mis-placed daemon (wrong NUMA node, unpinned memory) before a run is planned
on it.  The probe works INSIDE the slab (its first ``2 x mib`` MiB, before anything lives there): no extra pinned memory.
Role parity: reference ``src/dataflow/service/hostbw.py:13-47``.
"""
from __future__ import annotations

import time


def best_gbs(fn, payload_bytes: int, reps: int = 3) -> float:
    best = 0.0
    for _ in range(reps):
        t0 = time.perf_counter()
        fn()
        best = max(best, payload_bytes / max(time.perf_counter() - t0, 1e-9) / 1e9)
    return round(best, 2)


def measure_host_bw(slab, mib: int = 256, device: int | None = None) -> dict:
    """GB/s per lane, best of three; ``mib = 0`` (or a slab smaller than two payloads) disables the probe."""
    n = int(mib) << 20
    if n <= 0 or slab is None or slab.nbytes < 2 * n:
        return {}
    import numpy as np
    import torch
    a = torch.from_numpy(np.frombuffer(slab.bytes_view(0, n), dtype=np.uint8))
    b = torch.from_numpy(np.frombuffer(slab.bytes_view(n, n), dtype=np.uint8))
    a.fill_(1)
    b.fill_(2)
    out = {"host_copy_gbs": best_gbs(lambda: b.copy_(a), n)}
    x, y = a.view(torch.bfloat16), b.view(torch.bfloat16)
    x.add_(y)                                     # warm pages and the kernel
    out["host_bf16_add_gbs"] = best_gbs(lambda: x.add_(y), n)
    if device is not None and torch.cuda.is_available():
        d = torch.empty(n, dtype=torch.uint8, device=f"cuda:{device}")
        d.fill_(3)

        def sync_copy(dst, src):
            dst.copy_(src, non_blocking=True)
            torch.cuda.synchronize(device)
        torch.cuda.synchronize(device)
        out["h2d_gbs"] = best_gbs(lambda: sync_copy(d, a), n)
        out["d2h_gbs"] = best_gbs(lambda: sync_copy(a, d), n)
    a.zero_()
    b.zero_()
    return out
