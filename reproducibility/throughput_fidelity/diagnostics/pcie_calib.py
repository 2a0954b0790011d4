#!/usr/bin/env python
"""Host-link calibration: what a pinned-memory copy really costs, per direction, alone and with the other direction busy.

For sizes from 1 MiB to ``--max-mib`` the tool times host-to-device and device-to-host copies from pinned memory on a
stream of their own, then both directions at once on two streams, and fits ``time = latency + bytes / bandwidth`` per
direction and mode (least squares).  The planner prices every transfer with one bandwidth per direction; the fit says
which number to give it (``--h2d-gbs`` / ``--d2h-gbs`` of the tools, the ``pcie`` row of a hardware description) and how
much of a small transfer is latency.  Buffers are bounded by ``--max-mib`` (default 512); nothing else is touched.

    python reproducibility/throughput_fidelity/diagnostics/pcie_calib.py --device 0 --json pcie.json
"""
from __future__ import annotations

import argparse
import json
import sys


def fit(points: list[tuple[int, float]]) -> dict:
    """Least squares of seconds against bytes: returns latency (us) and bandwidth (GB/s)."""
    n = len(points)
    sx = sum(b for b, _ in points)
    sy = sum(t for _, t in points)
    sxx = sum(b * b for b, _ in points)
    sxy = sum(b * t for b, t in points)
    den = n * sxx - sx * sx
    if n < 2 or den == 0:
        return {"latency_us": 0.0, "gbs": 0.0}
    slope = (n * sxy - sx * sy) / den
    icpt = (sy - slope * sx) / n
    return {"latency_us": max(icpt, 0.0) * 1e6, "gbs": (1.0 / slope / 1e9) if slope > 0 else float("inf")}


def measure(device: int, max_mib: int, reps: int) -> dict:
    import torch
    torch.cuda.set_device(device)
    top = max_mib << 20
    host_a = torch.empty(top, dtype=torch.uint8).pin_memory()
    host_b = torch.empty(top, dtype=torch.uint8).pin_memory()
    dev_a = torch.empty(top, dtype=torch.uint8, device=device)
    dev_b = torch.empty(top, dtype=torch.uint8, device=device)
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def timed(n: int, h2d: bool, d2h: bool) -> float:
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        torch.cuda.synchronize()
        if h2d:
            with torch.cuda.stream(s_in):
                ev[0].record()
                for _ in range(reps):
                    dev_a[:n].copy_(host_a[:n], non_blocking=True)
                ev[1].record()
        if d2h:
            with torch.cuda.stream(s_out):
                ev[2].record()
                for _ in range(reps):
                    host_b[:n].copy_(dev_b[:n], non_blocking=True)
                ev[3].record()
        torch.cuda.synchronize()
        return max(ev[0].elapsed_time(ev[1]) if h2d else 0.0, ev[2].elapsed_time(ev[3]) if d2h else 0.0) / 1e3 / reps

    sizes = []
    n = 1 << 20
    while n <= top:
        sizes.append(n)
        n *= 4
    out = {"sizes_bytes": sizes, "h2d": [], "d2h": [], "both": []}
    for n in sizes:
        timed(n, True, True)                                       # warm-up
        out["h2d"].append(timed(n, True, False))
        out["d2h"].append(timed(n, False, True))
        out["both"].append(timed(n, True, True))
    out["fit"] = {k: fit(list(zip(sizes, out[k]))) for k in ("h2d", "d2h", "both")}
    big = sizes[-1]
    out["at_largest"] = {"h2d_gbs": big / out["h2d"][-1] / 1e9, "d2h_gbs": big / out["d2h"][-1] / 1e9,
                         "each_direction_when_both_gbs": big / out["both"][-1] / 1e9}
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--device", default="0")
    ap.add_argument("--max-mib", type=int, default=512)
    ap.add_argument("--reps", type=int, default=8)
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    import torch
    if a.device == "cpu" or not torch.cuda.is_available():
        res = {"device": "cpu", "note": "no device: nothing to calibrate"}
    else:
        res = measure(int(a.device), min(a.max_mib, 2048), a.reps)
        f = res["fit"]
        print(f"host to device: {f['h2d']['gbs']:.1f} GB/s + {f['h2d']['latency_us']:.0f} us;  device to host: {f['d2h']['gbs']:.1f} GB/s + "
              f"{f['d2h']['latency_us']:.0f} us;  both at once: {res['at_largest']['each_direction_when_both_gbs']:.1f} GB/s each")
    if a.json:
        with open(a.json, "w") as fh:
            json.dump(res, fh, indent=1)
    else:
        print(json.dumps(res if res.get("device") == "cpu" else res["fit"]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
