#!/usr/bin/env python
"""Times causal attention forward and backward on one GPU: this repository's tcgen05 kernels beside the vendor kernels of
the baseline lane (cuDNN fused attention for uniform rounds), with CUDA events after warm-up.

    python tools/bench/attention_bench.py --batch 4 --seq 4096 --hq 32 --hkv 8

Prints one JSON line: milliseconds and achieved TFLOP/s per implementation (causal FLOPs: 4 * T * S * hq * d / 2 forward,
2.5x that backward), and the largest difference between the two lanes' results.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", default=None, help="own | library: time one lane only (e.g. for a profiler capture)")
    ap.add_argument("--timeline", action="store_true",
                    help="print the forward kernel's own per-key-tile clock stamps (one CTA: its MMA thread and one softmax thread per query tile)")
    a = ap.parse_args(argv)
    import torch
    from dataflow_b200.ops import native, registered_ops, resolve_kernels
    from dataflow_b200.ops.cuda import flash_bwd_tcgen05, flash_fwd_tcgen05
    resolve_kernels()
    lib = {op: {k.name: k.fn for k in registered_ops()[op]}["baseline"] for op in ("flash_fwd", "flash_bwd")}
    B, S, HQ, HKV, D = a.batch, a.seq, a.hq, a.hkv, 128
    T = B * S
    g = torch.Generator(device="cuda").manual_seed(0)
    qkv = torch.randn(T, (HQ + 2 * HKV) * D, device="cuda", generator=g).bfloat16()
    q = qkv[:, :HQ * D].unflatten(1, (HQ, D))
    k = qkv[:, HQ * D:(HQ + HKV) * D].unflatten(1, (HKV, D))
    v = qkv[:, (HQ + HKV) * D:].unflatten(1, (HKV, D))
    do = torch.randn(T, HQ, D, device="cuda", generator=g).bfloat16()
    dqkv = torch.empty_like(qkv)
    dq = dqkv[:, :HQ * D].unflatten(1, (HQ, D))
    dk = dqkv[:, HQ * D:(HQ + HKV) * D].unflatten(1, (HKV, D))
    dv = dqkv[:, (HQ + HKV) * D:].unflatten(1, (HKV, D))
    cu = torch.arange(0, T + 1, S, device="cuda", dtype=torch.int32)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")          # larger than L2

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / a.iters

    if a.timeline:
        trace = torch.zeros(3 * 32 * 8, dtype=torch.int64, device="cuda")
        o = torch.empty(q.shape, dtype=q.dtype, device="cuda")
        lse = torch.empty(HQ, T, dtype=torch.float32, device="cuda")
        for _ in range(2):
            native().flash_fwd(q, k, v, o, lse, cu, S, D ** -0.5, trace)
        torch.cuda.synchronize()
        tr = trace.view(3, 32, 8).cpu()
        t0 = int(tr[tr > 0].min())
        names = ["softmax tile 0: wait S | S seen | loaded | max done | exp done | arrived",
                 "softmax tile 1: same", "MMA thread: [tile0: wait P | P seen | issued] [tile1: ...]"]
        for who in range(3):
            print(names[who])
            for j in range(2, 12):
                print("  j=%2d " % j + " ".join("%7d" % (int(x) - t0 if x > 0 else -1) for x in tr[who, j]))
        # the dK / dV kernel of the backward: math group 0 / 1 (wait S | S seen | loaded | math done | stored | arrived) and the
        # MMA thread (wait P | P seen | dV dK issued | next S^T dP^T issued)
        trace.zero_()
        scratch = torch.empty(2 * HQ * T, dtype=torch.float32, device="cuda")
        for _ in range(2):
            native().flash_bwd(do, q, k, v, o, lse, dq, dk, dv, scratch, cu, S, D ** -0.5, trace)
        torch.cuda.synchronize()
        tr = trace.view(3, 32, 8).cpu()
        t0 = int(tr[tr > 0].min())
        for who, name in enumerate(["dK/dV math group 0", "dK/dV math group 1", "dK/dV MMA thread"]):
            print(name)
            for j in range(4, 16):
                print("  it=%2d " % j + " ".join("%7d" % (int(x) - t0 if x > 0 else -1) for x in tr[who, j]))
        return 0
    fwd_flops = 4.0 * T * S * HQ * D / 2
    res = {"shape": {"batch": B, "seq": S, "hq": HQ, "hkv": HKV, "d": D}, "l2": "flushed between iterations"}
    if a.only != "library":
        o, lse = flash_fwd_tcgen05(q, k, v, cu, S)
        t = timed(lambda: flash_fwd_tcgen05(q, k, v, cu, S))
        res["own_fwd_ms"], res["own_fwd_tflops"] = t, fwd_flops / t / 1e9
        torch.cuda.synchronize()
        if native().gemm_last_error():
            raise SystemExit(f"the forward kernel raised error word {native().gemm_last_error()}")
        flash_bwd_tcgen05(do, q, k, v, o, lse, cu, S, dq=dq, dk=dk, dv=dv)
        torch.cuda.synchronize()
        if native().gemm_last_error():          # a kernel that gave up once would give up in every timed launch too
            raise SystemExit(f"the backward kernels raised error word {native().gemm_last_error()}")
        t = timed(lambda: flash_bwd_tcgen05(do, q, k, v, o, lse, cu, S, dq=dq, dk=dk, dv=dv))
        res["own_bwd_ms"], res["own_bwd_tflops"] = t, 2.5 * fwd_flops / t / 1e9
        res["error_word"] = native().gemm_last_error()
    if a.only != "own":
        o2, lse2 = lib["flash_fwd"](q, k, v, cu, S)
        t = timed(lambda: lib["flash_fwd"](q, k, v, cu, S))
        res["library_fwd_ms"], res["library_fwd_tflops"] = t, fwd_flops / t / 1e9
        g2 = lib["flash_bwd"](do, q, k, v, o2, lse2, cu, S)
        t = timed(lambda: lib["flash_bwd"](do, q, k, v, o2, lse2, cu, S))
        res["library_bwd_ms"], res["library_bwd_tflops"] = t, 2.5 * fwd_flops / t / 1e9
    if a.only is None:
        res["fwd_max_abs_diff"] = float((o.float() - o2.float()).abs().max())
        res["bwd_rel_diff"] = [float((x.float() - y.float()).norm() / y.float().norm()) for x, y in zip((dq, dk, dv), g2)]
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
