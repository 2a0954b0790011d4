"""Shared argument handling of the command-line tools: geometry grids, hardware overrides, table printing."""
from __future__ import annotations

import argparse
import dataclasses
import itertools
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def csv_ints(s: str) -> list[int]:
    return [int(x) for x in str(s).split(",") if x]


def csv_floats(s: str) -> list[float]:
    return [float(x) for x in str(s).split(",") if x]


def add_grid_flags(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--preset", default="llama3_8b", help="preset name or family:preset")
    ap.add_argument("--plugin", action="append", default=[], help="module that registers an external family")
    ap.add_argument("--t-round", default=None, help="tokens per round; a,b,c sweeps")
    ap.add_argument("--tokens-step", type=int, default=None, help="tokens per optimizer step (rounds = tokens-step / t-round)")
    ap.add_argument("--ga-rounds", type=int, default=None, help="gradient-accumulation rounds (alternative to --tokens-step)")
    ap.add_argument("--seq-len", default=None, help="sequence length; a,b,c sweeps")
    ap.add_argument("--budget", default=None, help="device budget GiB; a,b,c sweeps (default: unbounded)")
    ap.add_argument("--opt", default=None, choices=["adamw", "muon", "sgd", "sgdm"])
    ap.add_argument("--dtype-policy", default=None)
    ap.add_argument("--no-recompute", action="store_true")


def add_hw_flags(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--hw", default=None, help="hardware preset (default: the device found, else b200)")
    ap.add_argument("--tflops", type=float, default=None, help="override dense bf16 TFLOP/s")
    ap.add_argument("--bw", type=float, default=None, help="override device memory GB/s")
    ap.add_argument("--pcie", type=float, default=None, help="override host link GB/s (both directions)")


def hardware_from(a):
    from dataflow_b200.lowering.shaped_program import resolve_hardware
    hw = resolve_hardware(a.hw or "b200")
    kw = {}
    if a.tflops:
        kw["peak_tflops"] = a.tflops
    if a.bw:
        kw["hbm_gbs"] = a.bw
    if a.pcie:
        kw.update(h2d_gbs=a.pcie, d2h_gbs=a.pcie)
    return dataclasses.replace(hw, **kw) if kw else hw


def load_plugins(a) -> None:
    import importlib
    for m in a.plugin:
        importlib.import_module(m)


def grid_cells(a):
    """Yields ``(family, cfg, budget_gib)`` for every cell of the sweep."""
    from dataflow_b200.run.presets import resolve_preset
    load_plugins(a)
    fam, base = resolve_preset(a.preset)
    seqs = csv_ints(a.seq_len) if a.seq_len else [base.seq_len]
    trs = csv_ints(a.t_round) if a.t_round else [None]
    budgets = csv_floats(a.budget) if a.budget else [None]
    for s, tr, b in itertools.product(seqs, trs, budgets):
        t_round = tr if tr is not None else base.batch * s
        if t_round % s:
            raise SystemExit(f"--t-round {t_round} is not a multiple of --seq-len {s}")
        rounds = a.ga_rounds or (a.tokens_step // t_round if a.tokens_step else base.grad_accum_rounds)
        kw = {"seq_len": s, "batch": t_round // s, "grad_accum_rounds": max(int(rounds), 1)}
        if a.opt:
            kw["optimizer"] = a.opt
        if a.dtype_policy:
            kw["dtype_policy"] = a.dtype_policy
        yield fam, dataclasses.replace(base, **kw), b


def table(rows: list[dict], cols: list[tuple[str, str]]) -> str:
    """``cols``: (key, format) pairs; missing values print as '-'."""
    head = [k for k, _ in cols]
    body = [[(f.format(r[k]) if r.get(k) is not None else "-") for k, f in cols] for r in rows]
    w = [max(len(h), *(len(b[i]) for b in body)) if body else len(h) for i, h in enumerate(head)]
    lines = ["  ".join(h.rjust(w[i]) for i, h in enumerate(head))]
    lines += ["  ".join(c.rjust(w[i]) for i, c in enumerate(b)) for b in body]
    return "\n".join(lines)
