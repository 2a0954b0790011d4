"""The module library of the workload tracer: token mixers, feed-forward layers and the block that joins them, written as
``DataflowModule``s over the ops of ``ops.py``.  A module declares its parameters (global shapes; the tensor- and
expert-parallel layout of the context decides what one rank holds) and calls ops; everything the planner needs — FLOPs by
kind, bytes, saved activations, parameter counts — falls out of the trace.

    DenseAttention      grouped-query softmax attention, optional sliding window
    MLAAttention        multi-head latent attention (two low-rank stacks, decoupled rope key)
    DSAAttention        MLA projections + lightning indexer + attention over the selected keys in the latent form
    GatedDeltaNet       linear attention with a gated delta-rule state (short convolution, gated output norm)
    Mamba2Mixer         selective state-space mixer in its chunked form
    MLP                 SwiGLU (packed gate | up), GELU or squared-ReLU feed-forward
    MoE                 router, dispatch, grouped expert matmuls, combine, optional shared experts
    TransformerBlock    pre-norm residual block of one mixer and one feed-forward layer (either may be absent)
Reference role: ``src/dataflow_sim/workloads/modules/*.py``.
"""
from __future__ import annotations

from . import ops
from .tracing import DataflowModule, Sym, TraceContext


def _heads(t: Sym, h: int, d: int, name: str) -> Sym:
    return Sym(t.name + "." + name, (t.shape[0], h, d), t.dtype)


class DenseAttention(DataflowModule):
    name = "attn"

    def __init__(self, d_model: int, n_heads: int, n_kv_heads: int, head_dim: int, window: int = 0):
        self.d, self.hq, self.hkv, self.hd, self.window = d_model, n_heads, n_kv_heads, head_dim, window

    def forward(self, ctx: TraceContext, x: Sym) -> Sym:
        tp = ctx.tp
        hq, hkv = max(self.hq // tp, 1), max(self.hkv // tp, 1)
        x = ops.all_gather_rows(ctx, x, "ag")
        w_qkv = ctx.param("w_qkv", (self.d, (self.hq + 2 * self.hkv) * self.hd), shard="tp")
        qkv = ops.linear(ctx, x, w_qkv, "qkv")
        q = ops.rope(ctx, _heads(qkv, hq, self.hd, "q"), "rope_q")
        k = ops.rope(ctx, _heads(qkv, hkv, self.hd, "k"), "rope_k")
        v = _heads(qkv, hkv, self.hd, "v")
        o = ops.attention(ctx, q, k, v, "core", window=self.window)
        wo = ctx.param("wo", (self.hq * self.hd, self.d), shard="tp_rows")
        y = ops.linear(ctx, Sym(o.name, (o.shape[0], hq * self.hd), o.dtype), wo, "out")
        return ops.reduce_scatter_rows(ctx, y, "rs")


class MLAAttention(DataflowModule):
    name = "mla"

    def __init__(self, d_model: int, n_heads: int, q_lora: int, kv_lora: int, d_nope: int, d_rope: int, d_v: int):
        self.d, self.h, self.q_lora, self.kv_lora, self.dn, self.dr, self.dv = d_model, n_heads, q_lora, kv_lora, d_nope, d_rope, d_v

    def projections(self, ctx: TraceContext, x: Sym):
        """(q (T, h, dn + dr), normalised q latent, normalised kv latent + rope key (T, kv_lora + dr))."""
        h = max(self.h // ctx.tp, 1)
        x = ops.all_gather_rows(ctx, x, "ag")
        if self.q_lora:
            cq = ops.rmsnorm(ctx, ops.linear(ctx, x, ctx.param("wq_a", (self.d, self.q_lora)), "q_a"), "q_norm")
            q = ops.linear(ctx, cq, ctx.param("wq_b", (self.q_lora, self.h * (self.dn + self.dr)), shard="tp"), "q_b")
        else:
            cq = x
            q = ops.linear(ctx, x, ctx.param("wq", (self.d, self.h * (self.dn + self.dr)), shard="tp"), "q")
        kv_a = ops.linear(ctx, x, ctx.param("wkv_a", (self.d, self.kv_lora + self.dr)), "kv_a")
        latent = ops.rmsnorm(ctx, kv_a, "kv_norm", width=self.kv_lora)
        q = ops.rope(ctx, _heads(q, h, self.dn + self.dr, "heads"), "rope_q")
        return q, cq, latent

    def forward(self, ctx: TraceContext, x: Sym) -> Sym:
        h = max(self.h // ctx.tp, 1)
        q, _, latent = self.projections(ctx, x)
        ckv = Sym(latent.name + ".c", (latent.shape[0], self.kv_lora), latent.dtype)
        kv = ops.linear(ctx, ckv, ctx.param("wkv_b", (self.kv_lora, self.h * (self.dn + self.dv)), shard="tp"), "kv_b")
        k = Sym(kv.name + ".k", (kv.shape[0], h, self.dn + self.dr), kv.dtype)
        v = Sym(kv.name + ".v", (kv.shape[0], h, self.dv), kv.dtype)
        o = ops.attention(ctx, q, k, v, "core")
        wo = ctx.param("wo", (self.h * self.dv, self.d), shard="tp_rows")
        y = ops.linear(ctx, Sym(o.name, (o.shape[0], h * self.dv), o.dtype), wo, "out")
        return ops.reduce_scatter_rows(ctx, y, "rs")


class DSAAttention(MLAAttention):
    name = "dsa"

    def __init__(self, d_model, n_heads, q_lora, kv_lora, d_nope, d_rope, d_v, index_heads: int, index_dim: int, index_topk: int):
        super().__init__(d_model, n_heads, q_lora, kv_lora, d_nope, d_rope, d_v)
        self.hi, self.di, self.topk = index_heads, index_dim, index_topk

    def forward(self, ctx: TraceContext, x: Sym) -> Sym:
        h = max(self.h // ctx.tp, 1)
        q, cq, latent = self.projections(ctx, x)
        # lightning indexer: queries from the q latent, one shared LayerNorm'd key, per-head weights from the block input
        qi = ops.linear(ctx, cq, ctx.param("wi_q", (cq.shape[-1], self.hi * self.di)), "idx_q")
        ki = ops.rmsnorm(ctx, ops.linear(ctx, x, ctx.param("wi_k", (self.d, self.di)), "idx_k"), "idx_k_norm", bias=True)
        ops.linear(ctx, x, ctx.param("wi_w", (self.d, self.hi)), "idx_w", out_dtype="fp32")
        sel = ops.lightning_indexer(ctx, _heads(qi, self.hi, self.di, "heads"), ki, self.topk, "indexer")
        # latent form: W_kb folded into the query, values read from the latent, W_vb applied after the sum
        wkv_b = ctx.param("wkv_b", (self.kv_lora, self.h * (self.dn + self.dv)), shard="tp")
        t = x.shape[0]
        ctx.emit("absorb_q", "matmul", flops=2.0 * t * h * self.dn * self.kv_lora, bytes=q.nbytes + wkv_b.nbytes)
        ctx.emit("absorb_q.bwd", "matmul", flops=4.0 * t * h * self.dn * self.kv_lora, bytes=2.0 * q.nbytes + wkv_b.nbytes, phase="bwd")
        q_abs = ctx.tensor("q_abs", (t, h, self.kv_lora + self.dr))
        o_lat = ops.sparse_latent_attention(ctx, q_abs, latent, sel, self.kv_lora, "core")
        ctx.emit("expand_v", "matmul", flops=2.0 * t * h * self.kv_lora * self.dv, bytes=o_lat.nbytes + wkv_b.nbytes)
        ctx.emit("expand_v.bwd", "matmul", flops=4.0 * t * h * self.kv_lora * self.dv, bytes=2.0 * o_lat.nbytes + wkv_b.nbytes, phase="bwd")
        o = ctx.tensor("o", (t, h * self.dv))
        wo = ctx.param("wo", (self.h * self.dv, self.d), shard="tp_rows")
        return ops.reduce_scatter_rows(ctx, ops.linear(ctx, o, wo, "out"), "rs")


class GatedDeltaNet(DataflowModule):
    name = "gdn"

    def __init__(self, d_model: int, v_heads: int, k_heads: int, head_dim: int, state_dim: int, conv_width: int = 4):
        self.d, self.hv, self.hk, self.dv, self.dk, self.cw = d_model, v_heads, k_heads, head_dim, state_dim or head_dim, conv_width

    def forward(self, ctx: TraceContext, x: Sym) -> Sym:
        tp = ctx.tp
        hv, hk = max(self.hv // tp, 1), max(self.hk // tp, 1)
        x = ops.all_gather_rows(ctx, x, "ag")
        width = 2 * self.hk * self.dk + 2 * self.hv * self.dv + 2 * self.hv            # q, k | v, gate | beta, decay
        proj = ops.linear(ctx, x, ctx.param("w_in", (self.d, width), shard="tp"), "in")
        qkv = ops.causal_conv(ctx, Sym(proj.name + ".qkv", (proj.shape[0], 2 * hk * self.dk + hv * self.dv), proj.dtype), self.cw, "conv")
        rep = max(hv // hk, 1)
        q = Sym(qkv.name + ".q", (qkv.shape[0], hv, self.dk), qkv.dtype)               # k heads repeated to the v heads
        k = Sym(qkv.name + ".k", (qkv.shape[0], hv, self.dk), qkv.dtype)
        v = Sym(qkv.name + ".v", (qkv.shape[0], hv, self.dv), qkv.dtype)
        del rep
        o = ops.gated_delta_rule(ctx, q, k, v, "rule")
        on = ops.rmsnorm(ctx, Sym(o.name, (o.shape[0] * hv, self.dv), o.dtype), "o_norm")
        y = ops.linear(ctx, Sym(on.name, (x.shape[0], hv * self.dv), on.dtype), ctx.param("w_out", (self.hv * self.dv, self.d), shard="tp_rows"), "out")
        return ops.reduce_scatter_rows(ctx, y, "rs")


class Mamba2Mixer(DataflowModule):
    name = "mamba"

    def __init__(self, d_model: int, n_heads: int, n_groups: int, head_dim: int, state_dim: int, conv_width: int = 4):
        self.d, self.h, self.g, self.p, self.n, self.cw = d_model, n_heads, n_groups, head_dim, state_dim, conv_width

    def forward(self, ctx: TraceContext, x: Sym) -> Sym:
        tp = ctx.tp
        h, g = max(self.h // tp, 1), max(self.g // tp, 1)
        x = ops.all_gather_rows(ctx, x, "ag")
        width = 2 * self.h * self.p + 2 * self.g * self.n + self.h                     # x, z | B, C | dt
        proj = ops.linear(ctx, x, ctx.param("w_in", (self.d, width), shard="tp"), "in")
        xbc = ops.causal_conv(ctx, Sym(proj.name + ".xbc", (proj.shape[0], h * self.p + 2 * g * self.n), proj.dtype), self.cw, "conv")
        xs = Sym(xbc.name + ".x", (xbc.shape[0], h, self.p), xbc.dtype)
        b = Sym(xbc.name + ".b", (xbc.shape[0], g, self.n), xbc.dtype)
        c = Sym(xbc.name + ".c", (xbc.shape[0], g, self.n), xbc.dtype)
        o = ops.mamba2_scan(ctx, xs, b, c, "scan")
        on = ops.rmsnorm(ctx, Sym(o.name, (o.shape[0], h * self.p), o.dtype), "o_norm", width=self.h * self.p)
        y = ops.linear(ctx, on, ctx.param("w_out", (self.h * self.p, self.d), shard="tp_rows"), "out")
        return ops.reduce_scatter_rows(ctx, y, "rs")


class MLP(DataflowModule):
    name = "mlp"

    def __init__(self, d_model: int, d_ff: int, act: str = "swiglu"):
        self.d, self.f, self.act = d_model, d_ff, act

    def forward(self, ctx: TraceContext, x: Sym) -> Sym:
        gated = self.act == "swiglu"
        x = ops.all_gather_rows(ctx, x, "ag")
        w_up = ctx.param("w13" if gated else "w1", (self.d, (2 if gated else 1) * self.f), shard="tp")
        s = ops.gated_activation(ctx, ops.linear(ctx, x, w_up, "up"), self.act, gated=gated)
        y = ops.linear(ctx, s, ctx.param("w2", (self.f, self.d), shard="tp_rows"), "down", input_cheap=True)
        return ops.reduce_scatter_rows(ctx, y, "rs")


class MoE(DataflowModule):
    name = "moe"

    def __init__(self, d_model: int, n_experts: int, top_k: int, d_expert: int, n_shared: int = 0, act: str = "swiglu"):
        self.d, self.e, self.k, self.fe, self.shared, self.act = d_model, n_experts, top_k, d_expert, n_shared, act

    def forward(self, ctx: TraceContext, x: Sym) -> Sym:
        gated = self.act == "swiglu"
        ops.router(ctx, x, self.e, self.k, "router")
        xp = ops.moe_dispatch(ctx, x, self.k, "dispatch")
        share = self.k / self.e
        w_up = ctx.param("w13_experts", (self.e, self.d, (2 if gated else 1) * self.fe), shard="ep", active=share, kind="experts")
        s = ops.gated_activation(ctx, ops.grouped_linear(ctx, xp, w_up, "experts_up"), self.act, gated=gated)
        w_dn = ctx.param("w2_experts", (self.e, self.fe, self.d), shard="ep", active=share, kind="experts")
        yp = ops.grouped_linear(ctx, s, w_dn, "experts_down", input_cheap=True)
        y = ops.moe_combine(ctx, yp, x.shape[0], self.k, "combine")
        if self.shared:
            with ctx.scope("shared"):
                MLP(self.d, self.shared * self.fe, self.act).forward(ctx, x)
        return y


class TransformerBlock(DataflowModule):
    name = "block"

    def __init__(self, d_model: int, mixer: DataflowModule | None, ffn: DataflowModule | None, layernorm: bool = False):
        self.d, self.mixer, self.ffn, self.layernorm = d_model, mixer, ffn, layernorm

    def forward(self, ctx: TraceContext, x: Sym) -> Sym:
        for part, norm_name in ((self.mixer, "norm1"), (self.ffn, "norm2")):
            if part is None:
                continue
            h = ops.rmsnorm(ctx, x, norm_name, bias=self.layernorm)
            y = part(ctx, h)
            x = ops.residual_add(ctx, x, Sym(y.name, x.shape, x.dtype), norm_name + ".residual")
        return Sym(ctx.path("out"), x.shape, x.dtype)


def block_from_spec(layer, d_model: int) -> TransformerBlock:
    """The module for one ``LayerSpec`` (``builders.AttnSpec`` + ``builders.MlpSpec``)."""
    a, m = layer.attn, layer.mlp
    mixer: DataflowModule | None
    if a.kind == "none":
        mixer = None
    elif a.kind == "dense":
        mixer = DenseAttention(d_model, a.n_heads, a.n_kv_heads, a.head_dim, a.window)
    elif a.kind == "mla":
        mixer = MLAAttention(d_model, a.n_heads, a.q_lora, a.kv_lora, a.head_dim, a.rope_dim, a.v_head_dim or a.head_dim)
    elif a.kind == "dsa":
        mixer = DSAAttention(d_model, a.n_heads, a.q_lora, a.kv_lora, a.head_dim, a.rope_dim, a.v_head_dim or a.head_dim,
                             a.index_heads, a.index_dim, a.index_topk)
    elif a.kind == "linear":
        mixer = GatedDeltaNet(d_model, a.n_heads, a.n_kv_heads, a.head_dim, a.state_dim)
    elif a.kind == "mamba":
        mixer = Mamba2Mixer(d_model, a.n_heads, a.n_kv_heads, a.head_dim, a.state_dim)
    else:
        raise ValueError(f"unknown token mixer {a.kind!r}")
    ffn: DataflowModule | None
    if m.kind == "none":
        ffn = None
    elif m.kind == "moe":
        ffn = MoE(d_model, m.n_experts, m.top_k, m.d_expert, m.n_shared, m.expert_act)
    else:
        ffn = MLP(d_model, m.d_ff, m.kind)
    return TransformerBlock(d_model, mixer, ffn)
