#!/usr/bin/env python
"""Tensor-pipe step cost on this GPU: SM clocks per ``tcgen05.mma`` (128 x N x 16, bf16) by N and by where the operands come
from.  One CTA, one issuing thread, 256 instructions back to back; prints a table.

    python tools/bench/umma_probe.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main() -> int:
    import torch
    from dataflow_b200.ops import native
    kinds = ["A smem, B smem K-major", "A smem, B smem MN-major", "A tmem, B smem K-major", "A tmem, B smem MN-major"]
    count = 240
    print(f"{'operands':28s} {'N':>4s} {'accumulators':>13s} {'issue clk/instr':>16s} {'total clk/instr':>16s} {'ideal (4096 MAC/clk)':>22s}")
    for kind, name in enumerate(kinds):
        for n, naccs in ((64, (1, 2, 4)), (128, (1, 2, 3)), (256, (1,))):
            for nacc in naccs:
                native().umma_probe(kind, n, count, nacc)                      # warm-up
                r = native().umma_probe(kind, n, count, nacc)
                torch.cuda.synchronize()
                issue, total, bad = (int(x) for x in r.cpu())
                print(f"{name:28s} {n:4d} {nacc:13d} {issue / count:16.1f} {total / count:16.1f} {128 * n * 16 / 4096:22.1f}"
                      + ("  TIMED OUT" if bad else ""))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
