"""gpt2 family: LayerNorm (mean + rstd), fused c_attn QKV with bias, learned positions
(``[wte, wpe]`` in one embed object), GELU-tanh MLP, optional tied embedding / head, optional
bias-free variant, GPT-2 init policy (biases 0, residual projections N(0, 0.02/sqrt(2L))).
Activations follow ``act_dtype`` so the fp32 CPU configuration (124M, seq 1024, batch 2, ga 2)
runs end to end on the host backend.  Family parity: reference
``src/dataflow_training/model_families/gpt2/{model.py:39-272,blocks.py}``.
"""
from __future__ import annotations

from ...blocks.init_policy import set_init_layer

from dataclasses import dataclass
from typing import Any, Mapping

from ...blocks.layouts import DTypePolicy, Field, PackedLayout, grad_layout, opt_state_layout, weight_layout
from ...core import Program
from ...core.types import dtype_nbytes
from ...lowering.shaped_program import (LayerKindSpec, LooseCosts, ShapedConfig, ShapedHardware,
                                        build_shaped_program, optimizer_cost_seed, resolve_hardware)
from ..llama3.model import FamilyLayouts, _subop, init_field


@dataclass(frozen=True)
class ShapedGpt2Config:
    name: str = "gpt2"
    n_layers: int = 2
    d_model: int = 128
    n_heads: int = 4
    vocab_size: int = 512
    max_positions: int = 1024
    ln_eps: float = 1e-5
    seq_len: int = 64
    batch: int = 2
    grad_accum_rounds: int = 1
    tied_embeddings: bool = False
    bias: bool = True
    dtype_policy: Any = "bf16"
    act_dtype: str = "bf16"
    optimizer: str = "adamw"
    optimizer_placement: str = "interleaved"
    head_chunk_tokens: int = 2048
    family: str = "gpt2"

    @property
    def tokens_per_round(self) -> int:
        return self.seq_len * self.batch

    def policy(self) -> DTypePolicy:
        return self.dtype_policy if isinstance(self.dtype_policy, DTypePolicy) else DTypePolicy.from_dict(self.dtype_policy)


@dataclass(frozen=True)
class Gpt2Dims:
    n_layers: int
    d: int
    hq: int
    hd: int
    F: int
    vocab: int
    n_pos: int
    eps: float
    T: int
    seq_len: int
    head_chunk: int
    tied: bool
    bias: bool
    act: str = "bf16"

    @property
    def hkv(self) -> int:
        return self.hq


def derive_dims(cfg: ShapedGpt2Config) -> Gpt2Dims:
    return Gpt2Dims(cfg.n_layers, cfg.d_model, cfg.n_heads, cfg.d_model // cfg.n_heads, 4 * cfg.d_model, cfg.vocab_size,
                    max(cfg.max_positions, cfg.seq_len), cfg.ln_eps, cfg.tokens_per_round, cfg.seq_len,
                    min(cfg.head_chunk_tokens, cfg.tokens_per_round), cfg.tied_embeddings, cfg.bias, cfg.act_dtype)


def block_fields(d: Gpt2Dims) -> tuple[Field, ...]:
    f = [Field("ln1_w", (d.d,), "bf16", "vector", "ones")]
    if d.bias:
        f.append(Field("ln1_b", (d.d,), "bf16", "vector", "zeros"))
    f.append(Field("c_attn_w", (d.d, 3 * d.d), "bf16", "matrix", "normal"))
    if d.bias:
        f.append(Field("c_attn_b", (3 * d.d,), "bf16", "vector", "zeros"))
    f.append(Field("attn_proj_w", (d.d, d.d), "bf16", "matrix", "residual"))
    if d.bias:
        f.append(Field("attn_proj_b", (d.d,), "bf16", "vector", "zeros"))
    f.append(Field("ln2_w", (d.d,), "bf16", "vector", "ones"))
    if d.bias:
        f.append(Field("ln2_b", (d.d,), "bf16", "vector", "zeros"))
    f.append(Field("fc_w", (d.d, d.F), "bf16", "matrix", "normal"))
    if d.bias:
        f.append(Field("fc_b", (d.F,), "bf16", "vector", "zeros"))
    f.append(Field("mlp_proj_w", (d.F, d.d), "bf16", "matrix", "residual"))
    if d.bias:
        f.append(Field("mlp_proj_b", (d.d,), "bf16", "vector", "zeros"))
    return tuple(f)


def embed_fields(d: Gpt2Dims) -> tuple[Field, ...]:
    return (Field("wte", (d.vocab, d.d), "bf16", "embedding", "normal"),
            Field("wpe", (d.n_pos, d.d), "bf16", "embedding", "normal"))


def head_fields(d: Gpt2Dims) -> tuple[Field, ...]:
    f = [Field("final_norm", (d.d,), "bf16", "vector", "ones")]
    if d.bias:
        f.append(Field("final_norm_b", (d.d,), "bf16", "vector", "zeros"))
    if not d.tied:
        f.append(Field("w_head", (d.d, d.vocab), "bf16", "matrix", "normal"))
    return tuple(f)


def context_layout(d: Gpt2Dims, level: int = 0) -> PackedLayout:
    if level >= 2:
        return PackedLayout(())
    a = d.act
    f = [Field("mean1", (d.T,), "fp32"), Field("rstd1", (d.T,), "fp32"), Field("qkv", (d.T, 3 * d.d), a),
         Field("lse", (d.hq, d.T), "fp32"), Field("attn_out", (d.T, d.d), a), Field("h_mid", (d.T, d.d), a),
         Field("mean2", (d.T,), "fp32"), Field("rstd2", (d.T,), "fp32")]
    if level == 0:
        f.append(Field("fc", (d.T, d.F), a))
    return PackedLayout(tuple(f))


def family_layouts(d: Gpt2Dims, policy: DTypePolicy | None = None, optimizer: str = "adamw") -> FamilyLayouts:
    policy = policy or DTypePolicy.named("bf16")
    rule = lambda f: optimizer  # noqa: E731
    bf, ef, hf = block_fields(d), embed_fields(d), head_fields(d)
    return FamilyLayouts(
        d, policy,
        weight_layout(bf, policy), grad_layout(bf, policy), opt_state_layout(bf, policy, rule_of=rule),
        weight_layout(ef, policy), grad_layout(ef, policy), opt_state_layout(ef, policy, rule_of=rule),
        weight_layout(hf, policy), grad_layout(hf, policy), opt_state_layout(hf, policy, rule_of=rule),
        context_layout(d), {"Ap": context_layout(d, 1)})


def flops_per_token(cfg: ShapedGpt2Config) -> float:
    d = derive_dims(cfg)
    gemm = 2.0 * (d.d * 3 * d.d + d.d * d.d + 2 * d.d * d.F)
    attn = 2.0 * d.seq_len * d.d
    return 3.0 * (d.n_layers * (gemm + attn) + 2.0 * d.d * d.vocab) + 0.5 * d.n_layers * attn


def lower_gpt2(cfg: ShapedGpt2Config, recompute_levels: Mapping | None = None, hw: ShapedHardware | None = None,
               block_params: Mapping[str, Any] | None = None, comm_groups: Mapping[str, str] | None = None,
               zero: Mapping[str, Any] | None = None,
                 resident_params: bool = False) -> Program:
    hw = hw or resolve_hardware("b200")
    d = derive_dims(cfg)
    lay = family_layouts(d, cfg.policy(), cfg.optimizer)
    T, S = d.T, d.seq_len
    ab = dtype_nbytes(d.act, 1)
    gemm = 2.0 * T * (d.d * 3 * d.d + d.d * d.d + 2 * d.d * d.F)
    attn = 2.0 * S * T * d.d
    ew = float(ab) * T * (8 * d.d + 3 * d.F)
    fwd_us = hw.matmul_us(gemm) + hw.attn_us(attn) + hw.mem_us(ew)
    bwd_us = hw.matmul_us(2 * gemm) + hw.attn_us(2.5 * attn, True) + hw.mem_us(2.5 * ew)
    w, dw, o = lay.block_w.size_bytes, lay.block_dw.size_bytes, lay.block_o.size_bytes
    ws = T * (3 * d.d + 2 * d.F) * ab + (1 << 20)
    kind = LayerKindSpec("block", w, dw, o, lay.ctx.size_bytes, fwd_us, bwd_us, fwd_us,
                         optimizer_cost_seed(hw, w, dw, o, cfg.optimizer),
                         (_subop("gemms", gemm), _subop("attention", attn, eff="attention"), _subop("elementwise", nbytes=ew, eff="memory")),
                         (_subop("gemms", 2 * gemm), _subop("attention", 2.5 * attn, eff="attention_bwd"), _subop("elementwise", nbytes=2.5 * ew, eff="memory")),
                         (), (_subop("optimizer", nbytes=2 * w + dw + 2 * o, eff="memory"),), ws, 2 * ws, 0,
                         recompute_levels=((1, lay.extra["Ap"].size_bytes, hw.matmul_us(2.0 * T * d.d * d.F) + hw.mem_us(ew / 3)),
                                           (2, 0, fwd_us)))
    head_gemm = 2.0 * T * d.d * d.vocab
    loose = LooseCosts(hw.mem_us(2.0 * T * d.d * ab) + 5, hw.mem_us(4.0 * T * d.d * ab) + 30,
                       hw.matmul_us(3 * head_gemm) + hw.mem_us(3.0 * T * d.vocab * ab), 2.0,
                       (_subop("head_gemms", 3 * head_gemm),), d.head_chunk * d.vocab * ab + d.head_chunk * d.d * 8 + (1 << 20))
    sc = ShapedConfig(cfg.name, d.n_layers, T, cfg.grad_accum_rounds, d.d, ab, cfg.optimizer_placement, cfg.tied_embeddings)
    return build_shaped_program(
        sc, {"block": kind}, ["block"] * d.n_layers,
        embed_w_bytes=lay.embed_w.size_bytes, embed_dw_bytes=lay.embed_dw.size_bytes, embed_o_bytes=lay.embed_o.size_bytes,
        head_w_bytes=lay.head_w.size_bytes, head_dw_bytes=lay.head_dw.size_bytes, head_o_bytes=lay.head_o.size_bytes,
        loose=loose, hw=hw, recompute_levels=recompute_levels, block_params=block_params, comm_groups=comm_groups, zero=zero, resident_params=resident_params,
        metadata={"family": "gpt2", "preset": cfg.name, "flops_per_token": flops_per_token(cfg), "seq_len": cfg.seq_len,
                  "batch": cfg.batch})


def initial_values(program: Program, cfg: ShapedGpt2Config, views_of, seed: int = 0, layouts: FamilyLayouts | None = None) -> None:
    import torch
    d = derive_dims(cfg)
    lay = layouts or family_layouts(d, cfg.policy(), cfg.optimizer)
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    ids = {o.id for o in program.initial_objects}
    for oid in ["W_embed"] + [f"W_{i}" for i in range(d.n_layers)] + ["W_head"]:
        if oid not in ids:
            continue
        set_init_layer(oid)
        wl = lay.layout_of(oid)
        wv = views_of(oid, wl)
        for f in wl.fields:
            init_field(wv[f.name], f, gen, d.n_layers)
        oname = "O" + oid[1:]
        if oname in ids:
            ol = lay.layout_of(oname)
            ov = views_of(oname, ol)
            for f in ol.fields:
                if f.name.endswith(".master"):
                    ov[f.name].copy_(wv[f.name[:-7]].float())
                else:
                    ov[f.name].zero_()
