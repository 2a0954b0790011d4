"""Varlen segment descriptor of one round: ``cu_seqlens``, per-token ``positions`` that
restart at every packed sequence, the longest segment (a host int, never read back
from the device) and the content row count.  Resolved once per (run, round) from
``run_args["seq_lens"][round]`` — the boundary list ``[0, b1, …, content]`` — by the
first task that needs it.  Parity: reference ``src/dataflow_training/data/segments.py:18-232``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass
class Segments:
    cu_seqlens: Any        # int32 tensor (n_seq + 1) on the compute device
    positions: Any         # int32 tensor (n_tokens)
    bounds: tuple[int, ...]
    max_len: int
    n_tokens: int

    @property
    def n_seq(self) -> int:
        return len(self.bounds) - 1


def uniform_bounds(tokens: int, seq_len: int) -> list[int]:
    b = list(range(0, tokens, seq_len)) + [tokens]
    return b


def make_segments(bounds, device=None) -> Segments:
    import torch
    bounds = [int(b) for b in bounds]
    assert bounds and bounds[0] == 0 and all(a <= b for a, b in zip(bounds, bounds[1:])), bounds
    lens = [b - a for a, b in zip(bounds[:-1], bounds[1:])]
    n = bounds[-1]
    pos = torch.cat([torch.arange(l, dtype=torch.int32) for l in lens]) if lens else torch.zeros(0, dtype=torch.int32)
    cu = torch.tensor(bounds, dtype=torch.int32)
    if device is not None:
        dev = torch.device("cuda", device)
        cu, pos = cu.to(dev, non_blocking=True), pos.to(dev, non_blocking=True)
    return Segments(cu, pos, tuple(bounds), max(lens, default=0), n)


_uniform_cache: dict[tuple, Segments] = {}


def resolve_segments(ctx, round_index: int, max_tokens: int, seq_len: int, device=None) -> Segments:
    key = ("segments", round_index)
    seg = ctx.run_values.get(key)
    if seg is not None:
        return seg
    spec = (ctx.run_args.get("seq_lens") or {})
    bounds = spec.get(round_index, spec.get(str(round_index)))
    if bounds is None:
        ck = (max_tokens, seq_len, device)
        seg = _uniform_cache.get(ck)
        if seg is None:
            seg = _uniform_cache[ck] = make_segments(uniform_bounds(max_tokens, seq_len), device)
    else:
        if bounds[-1] > max_tokens:
            raise ValueError(f"round {round_index} holds {bounds[-1]} tokens, buffers are sized for {max_tokens}")
        seg = make_segments(bounds, device)
    ctx.run_values[key] = seg
    return seg
