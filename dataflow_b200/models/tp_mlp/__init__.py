"""tp_mlp family: the llama-style block under tensor + sequence parallelism inside one NVSwitch box.

Heads (``w_qkv`` columns, ``wo`` rows) and FFN columns (``w13``, ``w2`` rows) are split over ``tp`` ranks; the
residual stream is split by rows, so norms, the embedding and the loss see ``T / tp`` rows while attention and the
MLP see every row of this rank's heads / columns.  A block is four fused kernels forward (all-gather -> GEMM for
``w_qkv`` and ``w13``, GEMM -> reduce-scatter for ``wo`` and ``w2``) and four backward, all from
``parallel.tp.TpGroup``; the weight gradients of the column-parallel matrices reuse the operand the fused gather
assembled.  Gradients of replicated parameters (norm weights, embedding, head) are summed over the group in front
of their optimizer step.  Each rank runs its own engine program over its own shard; the programs are identical, so
every rank plans the same schedule and the collectives line up.

The reference's family of this name shards only the MLP and all-reduces its output through NCCL
(``src/dataflow_training/model_families/tp_mlp/``, ``llama3/blocks.py:91-128``).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping

from ...lowering.shaped_program import ShapedConfig, ShapedHardware, build_shaped_program, resolve_hardware
from ..families import ModelFamily, register_family
from ..llama3.model import (ShapedLlama3Config, block_kind_spec, derive_dims, family_layouts, flops_per_token, init_field, loose_costs)
from .blocks import build_tp_resolver


def derive_tp_dims(cfg: ShapedLlama3Config):
    """This rank's share of the model: local heads and FFN columns, all ``T`` rows in attention / MLP, ``Ts`` rows elsewhere."""
    d = derive_dims(cfg)
    p = int(cfg.tp)
    if d.moe or d.qk_norm:
        raise ValueError("tp_mlp covers the dense llama block")
    for what, v in (("n_heads", d.hq), ("n_kv_heads", d.hkv), ("d_ff", d.F), ("tokens per round", d.T)):
        if v % p:
            raise ValueError(f"{what} = {v} does not split over tp = {p}")
    shard = p if getattr(cfg, "vocab_parallel", False) else 1
    if d.vocab % shard:
        raise ValueError(f"vocab_size = {d.vocab} does not split over tp = {p}")
    return dataclasses.replace(d, hq=d.hq // p, hkv=d.hkv // p, F=d.F // p, tp=p, head_chunk=min(d.head_chunk, d.T // p), head_shard=shard)


def shard_dims(d):
    """Dims as the row-sharded executables (embedding, head + loss, optimizer) see them."""
    return dataclasses.replace(d, T=d.Ts, tp=1, head_chunk=min(d.head_chunk, d.Ts))


def lower_tp(cfg: ShapedLlama3Config, recompute_levels: Mapping[int, int] | None = None, hw: ShapedHardware | None = None,
             block_params: Mapping[str, Any] | None = None, comm_groups: Mapping[str, str] | None = None,
             resident_params: bool = False, **_ignored):
    hw = hw or resolve_hardware("b200")
    d = derive_tp_dims(cfg)
    lay = family_layouts(d, cfg.policy(), cfg.optimizer)
    kind = block_kind_spec(d, lay, hw, cfg.optimizer)
    # four collectives each way per block; the fused kernels hide most of the transfer behind the GEMM tiles
    exposed = 0.3 * 4 * hw.comm_us(d.T * d.d * 2 * (d.tp - 1) / d.tp) if d.tp > 1 else 0.0
    kind = dataclasses.replace(kind, fwd_us=kind.fwd_us + exposed, bwd_us=kind.bwd_us + 1.5 * exposed, recompute_us=kind.recompute_us + exposed)
    sc = ShapedConfig(cfg.name, d.n_layers, d.Ts, cfg.grad_accum_rounds, d.d, 2, cfg.optimizer_placement)
    return build_shaped_program(
        sc, {"block": kind}, ["block"] * d.n_layers,
        embed_w_bytes=lay.embed_w.size_bytes, embed_dw_bytes=lay.embed_dw.size_bytes, embed_o_bytes=lay.embed_o.size_bytes,
        head_w_bytes=lay.head_w.size_bytes, head_dw_bytes=lay.head_dw.size_bytes, head_o_bytes=lay.head_o.size_bytes,
        loose=loose_costs(shard_dims(d), lay, hw), hw=hw, recompute_levels=recompute_levels, block_params=block_params,
        comm_groups={"tp": "tp", **dict(comm_groups or {})}, resident_params=resident_params,
        metadata={"family": "tp_mlp", "preset": cfg.name, "flops_per_token": flops_per_token(cfg) / d.tp, "seq_len": cfg.seq_len,
                  "batch": cfg.batch, "tp": d.tp, "tokens_per_round_global": d.T})


def slice_for_rank(name: str, full, d_full, rank: int, p: int, head_shard: int = 1):
    """This rank's part of a full-model field (``d_full``: the unsharded dims)."""
    import torch
    hd = d_full.hd
    if name == "w_qkv":
        ql, kl = d_full.hq // p * hd, d_full.hkv // p * hd
        q0, k0, v0 = 0, d_full.q_dim, d_full.q_dim + d_full.kv_dim
        return torch.cat([full[:, q0 + rank * ql:q0 + (rank + 1) * ql], full[:, k0 + rank * kl:k0 + (rank + 1) * kl],
                          full[:, v0 + rank * kl:v0 + (rank + 1) * kl]], dim=1)
    if name == "wo":
        ql = d_full.hq // p * hd
        return full[rank * ql:(rank + 1) * ql]
    if name == "w13":
        fl = d_full.F // p
        return torch.cat([full[:, rank * fl:(rank + 1) * fl], full[:, d_full.F + rank * fl:d_full.F + (rank + 1) * fl]], dim=1)
    if name == "w2":
        fl = d_full.F // p
        return full[rank * fl:(rank + 1) * fl]
    if name == "w_head" and head_shard > 1:
        vl = d_full.vocab // head_shard
        return full[:, rank * vl:(rank + 1) * vl]
    return full


def initial_values_tp(program, cfg: ShapedLlama3Config, views_of, seed: int = 0, layouts=None, rank: int = 0) -> None:
    """The same bytes as the unsharded llama3 model of this seed, cut for ``rank``: every rank draws the full fields
    from the seeded generator in the canonical order and keeps its slice."""
    import torch
    d_full = derive_dims(cfg)
    d = derive_tp_dims(cfg)
    lay = layouts or family_layouts(d, cfg.policy(), cfg.optimizer)
    full_lay = family_layouts(d_full, cfg.policy(), cfg.optimizer)
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    ids = {o.id for o in program.initial_objects}
    for oid in ["W_embed"] + [f"W_{i}" for i in range(d.n_layers)] + ["W_head"]:
        if oid not in ids:
            continue
        wl, fl = lay.layout_of(oid), full_lay.layout_of(oid)
        wv = views_of(oid, wl)
        for f in fl.fields:
            t = torch.empty(tuple(f.shape), dtype=torch.float32)
            init_field(t, f, gen, d.n_layers)
            wv[f.name].copy_(slice_for_rank(f.name, t, d_full, rank, d.tp, d.head_shard).to(wv[f.name].dtype))
        oname = "O" + oid[1:]
        if oname in ids:
            ol = lay.layout_of(oname)
            ov = views_of(oname, ol)
            for f in ol.fields:
                if f.name.endswith(".master"):
                    ov[f.name].copy_(wv[f.name[:-7]].float())
                else:
                    ov[f.name].zero_()


PRESETS = {
    "tiny": dict(name="tiny", n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, d_ff=512, vocab_size=1024,
                 seq_len=128, batch=2, grad_accum_rounds=2, tp=2),
    "llama3_70b_tp8": dict(name="llama3_70b_tp8", n_layers=80, d_model=8192, n_heads=64, n_kv_heads=8, head_dim=128, d_ff=28672,
                           vocab_size=128256, seq_len=8192, batch=2, grad_accum_rounds=8, tp=8, dtype_policy="bf16_split_master"),
    # the same with the output projection's columns split over the group: 1/8 of the head matrix, gradient and optimizer state
    "llama3_70b_tp8_vp": dict(name="llama3_70b_tp8_vp", n_layers=80, d_model=8192, n_heads=64, n_kv_heads=8, head_dim=128, d_ff=28672,
                              vocab_size=128256, seq_len=8192, batch=2, grad_accum_rounds=8, tp=8, vocab_parallel=True,
                              dtype_policy="bf16_split_master"),
}

FAMILY = register_family(ModelFamily(
    name="tp_mlp", config_type=ShapedLlama3Config, derive_dims=derive_tp_dims, lower=lower_tp, initial_values=initial_values_tp,
    build_resolver=build_tp_resolver,
    family_layouts=lambda dims, policy=None, optimizer="adamw": family_layouts(dims, policy, optimizer),
    presets={k: (lambda kw=v: ShapedLlama3Config(**{**kw, "family": "tp_mlp"})) for k, v in PRESETS.items()},
    twin=None, bridge=None, block_kinds=("block",), flops_per_token=flops_per_token))
