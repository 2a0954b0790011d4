"""llama3 family: config, dims, byte-exact layouts, lowering, seeded init.

RMSNorm, GQA attention with rotate-half RoPE, SwiGLU MLP.  Weights are packed
B200-first: Q, K, V projections are one ``(d, (hq + 2 hkv) * hd)`` matrix and the
gate / up projections one ``(d, 2 F)`` matrix, so a block forward is four large
tcgen05 GEMMs instead of seven.  Saved context per token matches the reference's
(q, k, v, attn_out, h_mid, x1, x3 + statistics).  Family parity: reference
``src/dataflow_training/model_families/llama3/{model.py,blocks.py,presets.py}``.
"""
from __future__ import annotations

from ...blocks.init_policy import set_init_layer

from dataclasses import dataclass, field, replace
from typing import Any, Mapping

from ...blocks.layouts import (DTypePolicy, Field, PackedLayout, grad_layout, opt_state_layout, weight_layout)
from ...core import Program
from ...lowering.shaped_program import (LayerKindSpec, LooseCosts, ShapedConfig, ShapedHardware,
                                        build_shaped_program, optimizer_cost_seed, resolve_hardware)


@dataclass(frozen=True)
class ShapedLlama3Config:
    name: str = "llama3"
    n_layers: int = 2
    d_model: int = 256
    n_heads: int = 4
    n_kv_heads: int = 2
    head_dim: int = 64
    d_ff: int = 512
    vocab_size: int = 1024
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    seq_len: int = 128
    batch: int = 2                       # sequences per round
    grad_accum_rounds: int = 1
    dtype_policy: Any = "bf16"           # name or DTypePolicy dict
    optimizer: str = "adamw"
    optimizer_placement: str = "interleaved"
    head_chunk_tokens: int = 2048
    qk_norm: bool | str = False          # True: RMSNorm per head on q and k (qwen3); "full": over the whole q / k row (olmoe)
    family: str = "llama3"
    # mixture-of-experts MLP (olmoe / qwen3moe variants): n_experts > 0 replaces the dense SwiGLU MLP
    n_experts: int = 0
    top_k: int = 0
    d_ff_expert: int = 0
    routing_mode: str = "topk_then_softmax"
    aux_coef: float = 0.0                # load-balance loss coefficient (gradient injected analytically)
    # tensor + sequence parallelism (tp_mlp family): heads and FFN columns split over ``tp`` ranks, the residual
    # stream split by rows
    tp: int = 1
    # with tp > 1: split the output projection's vocabulary columns over the ranks too (softmax statistics are exchanged
    # instead of holding the whole matrix, its gradient and its optimizer state on every rank)
    vocab_parallel: bool = False
    # expert parallelism: experts split over ``ep`` ranks (each keeps its own tokens); dispatched matrices hold
    # ``ep_capacity`` times the balanced share of rows
    ep: int = 1
    ep_capacity: float = 2.0

    @property
    def tokens_per_round(self) -> int:
        return self.seq_len * self.batch

    @property
    def tokens_per_step(self) -> int:
        return self.tokens_per_round * self.grad_accum_rounds

    def policy(self) -> DTypePolicy:
        return self.dtype_policy if isinstance(self.dtype_policy, DTypePolicy) else DTypePolicy.from_dict(self.dtype_policy)


@dataclass(frozen=True)
class Llama3Dims:
    n_layers: int
    d: int
    hq: int
    hkv: int
    hd: int
    F: int
    vocab: int
    theta: float
    eps: float
    T: int                               # max tokens per round
    seq_len: int
    head_chunk: int
    qk_norm: bool | str = False
    E: int = 0                           # experts (0: dense MLP)
    topk: int = 0
    Fe: int = 0                          # expert FFN width
    routing_mode: str = "topk_then_softmax"
    aux_coef: float = 0.0
    tp: int = 1                          # > 1: hq / hkv / F are this rank's share; the residual stream holds Ts rows
    ep: int = 1                          # > 1: this rank holds E / ep experts and serves rows of every rank's tokens
    ep_capacity: float = 2.0
    head_shard: int = 1                  # > 1 (vocab-parallel head under tp): ``w_head`` holds vocab / head_shard columns

    @property
    def vocab_local(self) -> int:
        """Columns of the output projection this rank holds."""
        return self.vocab // self.head_shard

    @property
    def El(self) -> int:
        """Experts held by this rank."""
        return self.E // self.ep

    @property
    def Ts(self) -> int:
        """Rows of the residual stream this rank holds (sequence parallelism)."""
        return self.T // self.tp

    @property
    def moe(self) -> bool:
        return self.E > 0

    @property
    def Mp(self) -> int:
        """Rows of the dispatched (expert-major, tile-padded) activation matrix: the static worst case."""
        n = self.T * self.topk
        if self.ep > 1:
            # expert parallelism: room for ``ep_capacity`` times the balanced share (at most every slot of every rank)
            want = int(min(self.ep_capacity * n, self.ep * n))
            return (want + 255) // 256 * 256 + self.El * 256
        return (n + 255) // 256 * 256 + self.E * 256

    @property
    def qkv_dim(self) -> int:
        return (self.hq + 2 * self.hkv) * self.hd

    @property
    def q_dim(self) -> int:
        return self.hq * self.hd

    @property
    def kv_dim(self) -> int:
        return self.hkv * self.hd


def derive_dims(cfg: ShapedLlama3Config) -> Llama3Dims:
    assert cfg.n_heads % cfg.n_kv_heads == 0
    return Llama3Dims(cfg.n_layers, cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.d_ff, cfg.vocab_size,
                      cfg.rope_theta, cfg.rms_eps, cfg.tokens_per_round, cfg.seq_len,
                      min(cfg.head_chunk_tokens, cfg.tokens_per_round), cfg.qk_norm, cfg.n_experts, cfg.top_k,
                      cfg.d_ff_expert, cfg.routing_mode, cfg.aux_coef, ep=int(getattr(cfg, "ep", 1)),
                      ep_capacity=float(getattr(cfg, "ep_capacity", 2.0)))


# --------------------------------------------------------------------------- layouts
def block_fields(d: Llama3Dims) -> tuple[Field, ...]:
    f = [Field("attn_norm", (d.d,), "bf16", "vector", "ones"),
         Field("w_qkv", (d.d, d.qkv_dim), "bf16", "matrix", "normal")]
    if d.qk_norm:
        qn, kn = (d.q_dim, d.kv_dim) if d.qk_norm == "full" else (d.hd, d.hd)
        f += [Field("q_norm", (qn,), "bf16", "vector", "ones"), Field("k_norm", (kn,), "bf16", "vector", "ones")]
    f += [Field("wo", (d.q_dim, d.d), "bf16", "matrix", "normal"),
          Field("ffn_norm", (d.d,), "bf16", "vector", "ones")]
    if d.moe:
        f += [Field("w_router", (d.d, d.E), "bf16", "matrix", "normal"),
              Field("w13_experts", (d.El, d.d, 2 * d.Fe), "bf16", "matrix", "normal"),
              Field("w2_experts", (d.El, d.Fe, d.d), "bf16", "matrix", "normal")]
    else:
        f += [Field("w13", (d.d, 2 * d.F), "bf16", "matrix", "normal"),
              Field("w2", (d.F, d.d), "bf16", "matrix", "normal")]
    return tuple(f)


def embed_fields(d: Llama3Dims) -> tuple[Field, ...]:
    return (Field("wte", (d.vocab, d.d), "bf16", "embedding", "normal"),)


def head_fields(d: Llama3Dims) -> tuple[Field, ...]:
    return (Field("final_norm", (d.d,), "bf16", "vector", "ones"),
            Field("w_head", (d.d, d.vocab_local), "bf16", "matrix", "normal"))


def context_layout(d: Llama3Dims, level: int = 0) -> PackedLayout:
    """Saved context of one block.  Level 1 drops ``h13`` (two thirds of the bytes; rebuilt by one
    norm re-apply + one GEMM), level 2 saves nothing."""
    if level >= 2:
        return PackedLayout(())
    full = _context_layout_full(d)
    if level == 1:
        return PackedLayout(tuple(f for f in full.fields if f.name not in ("h13", "h13p")))
    return full


def _context_layout_full(d: Llama3Dims) -> PackedLayout:
    # with tensor parallelism the norms and the residual stream see this rank's rows only (Ts); the attention and
    # MLP intermediates see every row of this rank's heads / columns
    f = [Field("rstd_attn", (d.Ts,), "fp32"), Field("qkv", (d.T, d.qkv_dim), "bf16")]
    if d.qk_norm:
        per_row = (1, 1) if d.qk_norm == "full" else (d.hq, d.hkv)
        f += [Field("q_rstd", (d.T, per_row[0]), "fp32"), Field("k_rstd", (d.T, per_row[1]), "fp32"),
              Field("qk_pre", (d.T, d.q_dim + d.kv_dim), "bf16")]
    f += [Field("lse", (d.hq, d.T), "fp32"), Field("attn_out", (d.T, d.q_dim), "bf16"),
          Field("h_mid", (d.Ts, d.d), "bf16"), Field("rstd_ffn", (d.Ts,), "fp32")]
    if d.moe:
        # the routing decision and the padded expert-major row tables are context: recompute and backward never
        # re-route; h13p is the up-projection of the dispatched rows (expert-major)
        f += [Field("router_logits", (d.T, d.E), "bf16"), Field("route_w", (d.T, d.topk), "fp32"),
              Field("route_ids", (d.T, d.topk), "int32"), Field("row_of", (d.T, d.topk), "int32"),
              Field("row_src", (d.Mp,), "int32"), Field("offsets_pad", (d.El + 1,), "int32"),
              Field("tile_expert", (d.Mp // 256,), "int32"), Field("counts", (d.E,), "int32")]
        if d.ep > 1:
            # rows of other ranks' tokens are pulled again in the backward, which rebuilds h13p with them: only the
            # routing plan is context (row_of = the row every local slot got at its expert's owner)
            f.append(Field("row_w", (d.Mp,), "fp32"))
        else:
            f.append(Field("h13p", (d.Mp, 2 * d.Fe), "bf16"))
    else:
        f.append(Field("h13", (d.T, 2 * d.F), "bf16"))
    return PackedLayout(tuple(f))


@dataclass(frozen=True)
class FamilyLayouts:
    """All packed layouts of one model instance, keyed the way the lowering names objects."""
    dims: Any
    policy: DTypePolicy
    block_w: PackedLayout
    block_dw: PackedLayout
    block_o: PackedLayout
    embed_w: PackedLayout
    embed_dw: PackedLayout
    embed_o: PackedLayout
    head_w: PackedLayout
    head_dw: PackedLayout
    head_o: PackedLayout
    ctx: PackedLayout
    extra: Mapping[str, PackedLayout] = field(default_factory=dict)

    def object_layouts(self, program: Program) -> dict[str, PackedLayout]:
        out: dict[str, PackedLayout] = {}
        for oid in program.object_sizes():
            lay = self.layout_of(oid)
            if lay is not None:
                out[oid] = lay
        return out

    def layout_of(self, oid: str) -> PackedLayout | None:
        if oid == "W_embed":
            return self.embed_w
        if oid == "O_embed":
            return self.embed_o
        if oid == "W_head":
            return self.head_w
        if oid == "O_head":
            return self.head_o
        if oid.startswith("dW_embed"):
            return self.embed_dw
        if oid.startswith("dW_head"):
            return self.head_dw
        if oid.startswith("W_"):
            return self.block_w
        if oid.startswith("O_"):
            return self.block_o
        if oid.startswith("dW_"):
            return self.block_dw
        if oid.startswith("A_"):
            return self.ctx
        if oid.startswith("Ap_"):
            return self.extra.get("Ap")
        return self.extra.get(oid.split("_")[0])


def family_layouts(d: Llama3Dims, policy: DTypePolicy | None = None, optimizer: str = "adamw") -> FamilyLayouts:
    policy = policy or DTypePolicy.named("bf16")
    rule = lambda f: optimizer  # noqa: E731
    bf, ef, hf = block_fields(d), embed_fields(d), head_fields(d)
    return FamilyLayouts(
        d, policy,
        weight_layout(bf, policy), grad_layout(bf, policy), opt_state_layout(bf, policy, rule_of=rule),
        weight_layout(ef, policy), grad_layout(ef, policy), opt_state_layout(ef, policy, rule_of=rule),
        weight_layout(hf, policy), grad_layout(hf, policy), opt_state_layout(hf, policy, rule_of=rule),
        context_layout(d), {"Ap": context_layout(d, 1)})


# --------------------------------------------------------------------------- cost seeds
def _subop(name, flops=0.0, nbytes=0.0, eff="matmul", dtype="bf16"):
    return {"name": name, "flops": float(flops), "memory_bytes": float(nbytes), "efficiency": eff, "dtype": dtype}


def block_kind_spec(d: Llama3Dims, lay: FamilyLayouts, hw: ShapedHardware, optimizer: str = "adamw") -> LayerKindSpec:
    T, S = d.T, d.seq_len
    mlp = (d.d * d.E + d.topk * (d.d * 2 * d.Fe + d.Fe * d.d)) if d.moe else (d.d * 2 * d.F + d.F * d.d)
    gemm = 2.0 * T * (d.d * d.qkv_dim + d.q_dim * d.d + mlp)
    attn = 2.0 * S * T * d.hd * d.hq            # causal: half of 4*S*T*hd*hq
    ffw = d.topk * (2 * d.Fe + 2 * d.d) if d.moe else 2 * d.F
    ew_bytes = 2.0 * T * (6 * d.d + 2 * d.qkv_dim + 3 * ffw)
    fwd_sub = (_subop("gemms", gemm), _subop("attention", attn, eff="attention"), _subop("elementwise", nbytes=ew_bytes, eff="memory"))
    bwd_sub = (_subop("gemms", 2 * gemm), _subop("attention", 2.5 * attn, eff="attention_bwd"),
               _subop("elementwise", nbytes=2.5 * ew_bytes, eff="memory"))
    fwd_us = hw.matmul_us(gemm) + hw.attn_us(attn) + hw.mem_us(ew_bytes)
    bwd_us = hw.matmul_us(2 * gemm) + hw.attn_us(2.5 * attn, True) + hw.mem_us(2.5 * ew_bytes)
    w, dw, o = lay.block_w.size_bytes, lay.block_dw.size_bytes, lay.block_o.size_bytes
    if d.moe:
        ws_f = d.Mp * (2 * d.d + d.Fe) * 2 + T * d.qkv_dim * 2 + (1 << 20)
        ws_b = d.Mp * (3 * d.d + 2 * d.Fe * 2 + d.Fe) * 2 + T * (d.qkv_dim + 3 * d.d) * 2 + (1 << 20)
    else:
        ws_f = T * max(d.qkv_dim, 2 * d.F) * 2 + (1 << 20)
        ws_b = T * (2 * d.F * 2 + d.F + d.qkv_dim + 2 * d.d) * 2 + (1 << 20)
    return LayerKindSpec(
        "block", w, dw, o, lay.ctx.size_bytes, fwd_us, bwd_us, fwd_us, optimizer_cost_seed(hw, w, dw, o, optimizer),
        fwd_sub, bwd_sub, fwd_sub, (_subop("optimizer", nbytes=2 * w + dw + 2 * o, eff="memory"),),
        ws_f, ws_b, 0,
        recompute_levels=(((1, lay.extra["Ap"].size_bytes,
                            hw.matmul_us(2.0 * T * d.d * (2 * d.Fe * d.topk if d.moe else 2 * d.F)) + hw.mem_us(ew_bytes / 3)),)
                          if d.ep == 1 else ()) + ((2, 0, fwd_us),))


def loose_costs(d: Llama3Dims, lay: FamilyLayouts, hw: ShapedHardware) -> LooseCosts:
    T = d.T
    head_gemm = 2.0 * T * d.d * d.vocab
    head_us = hw.matmul_us(3 * head_gemm) + hw.mem_us(3.0 * T * d.vocab * 2)
    ws = d.head_chunk * d.vocab * 2 + d.head_chunk * d.d * 4 + (1 << 20)
    return LooseCosts(hw.mem_us(2.0 * T * d.d * 2) + 5, hw.mem_us(4.0 * T * d.d * 2) + 30, head_us, 2.0,
                      (_subop("head_gemms", 3 * head_gemm), _subop("ce", nbytes=3.0 * T * d.vocab * 2, eff="memory")), ws)


def flops_per_token(cfg: ShapedLlama3Config) -> float:
    """Effective training FLOPs per token (fwd + bwd, causal attention counted at half)."""
    d = derive_dims(cfg)
    mlp = (d.d * d.E + d.topk * (d.d * 2 * d.Fe + d.Fe * d.d)) if d.moe else (d.d * 2 * d.F + d.F * d.d)
    gemm = 2.0 * (d.d * d.qkv_dim + d.q_dim * d.d + mlp)
    attn = 2.0 * d.seq_len * d.hd * d.hq
    return 3.0 * (d.n_layers * (gemm + attn) + 2.0 * d.d * d.vocab) + 0.5 * d.n_layers * attn


# --------------------------------------------------------------------------- lowering
def lower_llama3(cfg: ShapedLlama3Config, recompute_levels: Mapping[int, int] | None = None,
                 hw: ShapedHardware | None = None, block_params: Mapping[str, Any] | None = None,
                 comm_groups: Mapping[str, str] | None = None, zero: Mapping[str, Any] | None = None,
                 resident_params: bool = False) -> Program:
    hw = hw or resolve_hardware("b200")
    d = derive_dims(cfg)
    lay = family_layouts(d, cfg.policy(), cfg.optimizer)
    kind = block_kind_spec(d, lay, hw, cfg.optimizer)
    sc = ShapedConfig(cfg.name, d.n_layers, d.T, cfg.grad_accum_rounds, d.d, 2, cfg.optimizer_placement)
    return build_shaped_program(
        sc, {"block": kind}, ["block"] * d.n_layers,
        embed_w_bytes=lay.embed_w.size_bytes, embed_dw_bytes=lay.embed_dw.size_bytes, embed_o_bytes=lay.embed_o.size_bytes,
        head_w_bytes=lay.head_w.size_bytes, head_dw_bytes=lay.head_dw.size_bytes, head_o_bytes=lay.head_o.size_bytes,
        loose=loose_costs(d, lay, hw), hw=hw, recompute_levels=recompute_levels, block_params=block_params,
        comm_groups=({"ep": "ep", **dict(comm_groups or {})} if d.ep > 1 else comm_groups), zero=zero, resident_params=resident_params,
        metadata={"family": cfg.family, "preset": cfg.name, "flops_per_token": flops_per_token(cfg),
                  "seq_len": cfg.seq_len, "batch": cfg.batch, **({"ep": d.ep} if d.ep > 1 else {})})


# --------------------------------------------------------------------------- init
def init_field(t, f: Field, gen, n_layers: int, std: float = 0.02) -> None:
    """Fill tensor ``t`` (any dtype) for field ``f`` from the seeded CPU generator."""
    import torch
    from ...blocks.init_policy import fill_by_policy
    if fill_by_policy(t, f.name, gen):            # a run-level init policy (blocks/init_policy.py) names a rule for this field
        return
    if f.init == "ones":
        t.fill_(1.0)
    elif f.init == "zeros":
        t.zero_()
    else:
        s = std / (2 * n_layers) ** 0.5 if f.init == "residual" else std
        # sequential field order from one generator: the same seed gives the same bytes everywhere
        step = 1 << 24
        flat = t.reshape(-1)
        for lo in range(0, flat.numel(), step):
            n = min(step, flat.numel() - lo)
            flat[lo:lo + n].copy_(torch.empty(n, dtype=torch.float32).normal_(0.0, s, generator=gen))


def initial_values(program: Program, cfg: ShapedLlama3Config, views_of, seed: int = 0, layouts: FamilyLayouts | None = None,
                   rank: int = 0) -> None:
    """Write seeded initial parameters and optimizer state.  ``views_of(object_id, layout)`` returns
    name → tensor views over that object's backing bytes.  Under expert parallelism every rank draws the full expert
    stacks from the seeded generator and keeps the experts it owns (``rank``)."""
    import torch
    d = derive_dims(cfg)
    lay = layouts or family_layouts(d, cfg.policy(), cfg.optimizer)
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    order = ["W_embed"] + [f"W_{i}" for i in range(d.n_layers)] + ["W_head"]
    ids = {o.id for o in program.initial_objects}
    for oid in order:
        if oid not in ids:
            continue
        set_init_layer(oid)
        wl = lay.layout_of(oid)
        wv = views_of(oid, wl)
        for f in wl.fields:
            if d.ep > 1 and f.name in ("w13_experts", "w2_experts"):
                full = torch.empty((d.E,) + tuple(f.shape[1:]), dtype=torch.float32)
                init_field(full, f, gen, d.n_layers)
                wv[f.name].copy_(full[rank * d.El:(rank + 1) * d.El].to(wv[f.name].dtype))
            else:
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
