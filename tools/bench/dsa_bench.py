#!/usr/bin/env python
"""Times the sparse-attention indexer kernels on one GPU: index scores on tcgen05 and the top-k row selection, beside the
eager forms of the same ops (the (heads, queries, keys) intermediate of the eager scores limits its block of rows).

    python tools/bench/dsa_bench.py --seq 16384 --heads 64 --dim 128 --topk 2048

Prints one JSON line.  FLOPs of the scores: 2 * heads * dim per visible (query, key) pair of the timed block of rows; the
kernel computes whole 128 x 128 tiles, so tiles on the diagonal do about twice the counted work.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=16384)
    ap.add_argument("--heads", type=int, default=64)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--topk", type=int, default=2048)
    ap.add_argument("--rows", type=int, default=1024, help="query rows per launch (the last block of the sequence is timed)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--only", default=None, help="own: skip the eager forms (e.g. for a profiler capture)")
    a = ap.parse_args(argv)
    import torch
    from dataflow_b200.ops import eager, resolve_kernels
    K = resolve_kernels()
    n, H, D = a.seq, a.heads, a.dim
    g = torch.Generator(device="cuda").manual_seed(0)
    q = (torch.randn(n, H, D, device="cuda", generator=g) * D ** -0.25).bfloat16()
    k = (torch.randn(n, D, device="cuda", generator=g) * D ** -0.25).bfloat16()
    w = torch.randn(n, H, device="cuda", generator=g)
    start = torch.zeros(n, dtype=torch.int32, device="cuda")
    q0, q1 = n - a.rows, n
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / iters

    pairs = sum(i + 1 for i in range(q0, q1))
    flops = 2.0 * H * D * pairs
    out = {"shape": {"seq": n, "heads": H, "dim": D, "topk": a.topk, "rows": a.rows}, "l2": "flushed between iterations"}
    ms = timed(lambda: K.dsa_index_scores(q, k, w, start, q0, q1, 0), a.iters)
    out["scores_ms"] = ms
    out["scores_tflops"] = flops / ms / 1e9
    s = K.dsa_index_scores(q, k, w, start, q0, q1, 0)
    out["topk_ms"] = timed(lambda: K.dsa_topk_rows(s, a.topk, 0), a.iters)
    out["full_sequence_estimate_ms"] = {"scores": ms * (n / a.rows) * (sum(i + 1 for i in range(n)) / (pairs * n / a.rows)),
                                        "topk": out["topk_ms"] * n / a.rows}
    if a.only != "own":
        rows_e = min(a.rows, 128)             # the eager form holds (rows, heads, keys) fp32
        ms_e = timed(lambda: eager.dsa_index_scores(q, k, w, start, n - rows_e, n, 0), max(a.iters // 2, 1))
        out["eager_scores_ms_per_block_of_rows"] = ms_e * a.rows / rows_e
        out["eager_topk_ms"] = timed(lambda: eager.dsa_topk_rows(s, a.topk, 0), max(a.iters // 2, 1))
        ref = eager.dsa_index_scores(q, k, w, start, n - rows_e, n, 0)
        fin = torch.isfinite(ref)
        got = s[-rows_e:]
        out["scores_rel_diff"] = float((got[fin] - ref[fin]).norm() / ref[fin].norm())
        out["topk_equal"] = bool(torch.equal(K.dsa_topk_rows(s, a.topk, 0), eager.dsa_topk_rows(s, a.topk, 0)))
    from dataflow_b200.ops import native
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
