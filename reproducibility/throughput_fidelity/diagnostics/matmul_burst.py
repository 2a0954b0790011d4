#!/usr/bin/env python
"""GEMM throughput as a burst and sustained: a short run of bf16 GEMMs from idle, then the same GEMM for ``--seconds``
while the clocks are sampled (read only).  A kernel timed alone sees the burst figure, a kernel inside a long step the
sustained one; the gap between them (the power cap pulling the SM clock down) is what a per-task profile taken from short
runs over-promises, which is why task profiling soaks the device before it samples.

    python reproducibility/throughput_fidelity/diagnostics/matmul_burst.py --device 0 --seconds 8
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run(device: int, m: int, seconds: float) -> dict:
    import torch
    from stages.sweep import ClockSampler
    torch.cuda.set_device(device)
    x = torch.randn(m, m, dtype=torch.bfloat16, device=device)
    y = torch.randn(m, m, dtype=torch.bfloat16, device=device)
    flop = 2.0 * m ** 3

    def batch(k: int) -> float:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(k):
            torch.mm(x, y)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 1e3 / k

    batch(3)
    time.sleep(2.0)                                                # let the device idle: the burst starts from rest
    burst = flop / batch(10) / 1e12
    series = []
    with ClockSampler(device, period=0.25) as clocks:
        t_end = time.time() + seconds
        while time.time() < t_end:
            series.append(flop / batch(20) / 1e12)
    tail = series[len(series) // 2:] or series
    return {"m": m, "burst_tflops": burst, "sustained_tflops": sum(tail) / len(tail), "first_tflops": series[0], "last_tflops": series[-1],
            "clocks": clocks.summary(), "series_tflops": [round(v, 1) for v in series]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--device", default="0")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--seconds", type=float, default=8.0)
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    import torch
    if a.device == "cpu" or not torch.cuda.is_available():
        res = {"device": "cpu", "note": "no device"}
    else:
        res = run(int(a.device), min(a.m, 16384), min(a.seconds, 30.0))
        print(f"burst {res['burst_tflops']:.0f} TFLOP/s, sustained {res['sustained_tflops']:.0f} TFLOP/s "
              f"({100 * res['sustained_tflops'] / res['burst_tflops']:.0f} %), clocks {res['clocks']}")
    if a.json:
        with open(a.json, "w") as f:
            json.dump(res, f, indent=1)
    else:
        print(json.dumps({k: v for k, v in res.items() if k != "series_tflops"}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
