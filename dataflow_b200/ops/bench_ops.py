"""Micro-benchmarks of the hand-written kernels (CUDA events, L2 flushed between iterations).

    python -m dataflow_b200.ops.bench_ops gemm --m 8192 --n 8192 --k 8192 --layout nt --iters 20
    python -m dataflow_b200.ops.bench_ops gemm --m 4096 --n 4096 --k 4096 --iters 3 --no-compare   # small case for ncu

Prints achieved TFLOP/s (or GB/s) and the fraction of the measured device peak
(``MEASURED_PEAKS.json`` at the repository root when present).
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def peaks() -> dict:
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        return json.load(open(p))
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "fallback": True}


def time_fn(fn, iters: int, flush_mib: int = 256) -> float:
    flush = torch.empty(flush_mib << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def bench_gemm(a) -> None:
    from dataflow_b200.ops import native
    ops = native()
    a_mn, b_mn = a.layout[0] == "t", a.layout[1] == "n"
    A = torch.randn((a.k, a.m) if a_mn else (a.m, a.k), device="cuda").bfloat16()
    B = torch.randn((a.k, a.n) if b_mn else (a.n, a.k), device="cuda").bfloat16()
    D = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    ms = time_fn(lambda: ops.gemm_bf16(A, a_mn, B, b_mn, D, None, None), a.iters)
    fl = 2.0 * a.m * a.n * a.k
    pk = peaks()
    line = {"op": "gemm_bf16", "m": a.m, "n": a.n, "k": a.k, "layout": a.layout, "ms": ms, "tflops": fl / ms / 1e9,
            "frac_of_measured_cublas": fl / ms / 1e9 / pk["bf16_tflops"], "err": ops.gemm_last_error()}
    if not a.no_compare:
        Aop, Bop = (A.t() if a_mn else A), (B if b_mn else B.t())
        ref = time_fn(lambda: torch.matmul(Aop, Bop, out=D), a.iters)
        line["cublas_ms"], line["cublas_tflops"] = ref, fl / ref / 1e9
    print(json.dumps(line))


def bench_stream(a) -> None:
    """Memory-bound kernels against the measured copy bandwidth."""
    from dataflow_b200.ops import resolve_kernels
    K = resolve_kernels()
    rows, cols = a.m, a.n
    x = torch.randn(rows, cols, device="cuda").bfloat16()
    w = torch.ones(cols, device="cuda", dtype=torch.bfloat16)
    y = torch.empty_like(x)
    pk = peaks()
    ms = time_fn(lambda: K.rmsnorm_fwd(x, w, 1e-5, out=y), a.iters)
    gbs = 2.0 * x.numel() * 2 / ms / 1e6
    print(json.dumps({"op": "rmsnorm_fwd", "rows": rows, "cols": cols, "ms": ms, "gbs": gbs, "frac_of_measured_copy": gbs / pk["hbm_gbs"]}))
    h13 = torch.randn(rows, 2 * cols, device="cuda").bfloat16()
    s = torch.empty(rows, cols, device="cuda", dtype=torch.bfloat16)
    ms = time_fn(lambda: K.swiglu_packed_fwd(h13, out=s), a.iters)
    gbs = 3.0 * rows * cols * 2 / ms / 1e6
    print(json.dumps({"op": "swiglu_packed_fwd", "rows": rows, "F": cols, "ms": ms, "gbs": gbs, "frac_of_measured_copy": gbs / pk["hbm_gbs"]}))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemm", "stream"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--layout", default="nn", help="A then B: n = as stored for x @ W (A (M,K), B (K,N)); t = transposed storage")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-compare", action="store_true")
    a = ap.parse_args(argv)
    (bench_gemm if a.op == "gemm" else bench_stream)(a)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
