"""llama3 block executables: staged forward, derived recompute, backward, resolver.

The forward is an ordered list of stages ``(name, fn, emitted_context_fields)``;
saved context is written *through* into the ``A`` object as it is produced, and the
recompute task is derived — it runs the same stages up to the last one that emits
context.  Backward re-applies both norms from saved statistics and recomputes the
SwiGLU product instead of saving them.  Structure parity: reference
``src/dataflow_training/model_families/llama3/blocks.py:132-619``.
"""
from __future__ import annotations

from typing import Any, Mapping

from ...blocks.base_blocks import _Base, common_executables


# --------------------------------------------------------------------------- stages
def _lin(K, st):
    """The forward linear of the four large dense projections: bf16, or e4m3 operands with fp32 accumulation when the
    training configuration asks for ``linear_precision: fp8`` (backward GEMMs stay bf16; router logits stay bf16)."""
    return K.linear_fwd_fp8 if st.get("fp8") else K.linear_fwd_bf16


def stage_attn_norm(K, d, st):
    st["h"], rstd = K.rmsnorm_fwd(st["x"], st["w"]["attn_norm"], d.eps)
    st["a"]["rstd_attn"].copy_(rstd)


def _qkv_views(d, qkv, n):
    q = qkv[:, :d.q_dim].unflatten(1, (d.hq, d.hd))
    k = qkv[:, d.q_dim:d.q_dim + d.kv_dim].unflatten(1, (d.hkv, d.hd))
    v = qkv[:, d.q_dim + d.kv_dim:].unflatten(1, (d.hkv, d.hd))
    return q, k, v


def _norm_rows(d, t):
    """(tokens, heads, head_dim) -> the contiguous 2-D matrix whose rows the q / k RMSNorm normalises."""
    t = t.contiguous()
    return t.view(t.shape[0], -1) if d.qk_norm == "full" else t.view(-1, d.hd)


def stage_qkv_rope(K, d, st):
    qkv = st["a"]["qkv"]
    _lin(K, st)(st["h"], st["w"]["w_qkv"], out=qkv)
    q, k, v = _qkv_views(d, qkv, st["n"])
    if d.qk_norm:
        a = st["a"]
        a["qk_pre"].copy_(qkv[:, :d.q_dim + d.kv_dim])
        # rows of the norm: one head ("per head") or the whole projected row ("full")
        qrows, krows = _norm_rows(d, q), _norm_rows(d, k)
        qn, qr = K.rmsnorm_fwd(qrows, st["w"]["q_norm"], d.eps)
        kn, kr = K.rmsnorm_fwd(krows, st["w"]["k_norm"], d.eps)
        q.copy_(qn.view_as(q))
        k.copy_(kn.view_as(k))
        a["q_rstd"].copy_(qr.view(a["q_rstd"].shape))
        a["k_rstd"].copy_(kr.view(a["k_rstd"].shape))
    pos = st["seg"].positions
    K.rope_fwd(q, pos, d.theta)
    K.rope_fwd(k, pos, d.theta)
    st["q"], st["k"], st["v"] = q, k, v


def stage_attn(K, d, st):
    seg = st["seg"]
    out = st["a"]["attn_out"].unflatten(1, (d.hq, d.hd))
    _, lse = K.flash_fwd(st["q"], st["k"], st["v"], seg.cu_seqlens, seg.max_len, out=out)
    st["a"]["lse"].copy_(lse)


def stage_resid1_norm2(K, d, st):
    h_mid = st["a"]["h_mid"]
    _lin(K, st)(st["a"]["attn_out"], st["w"]["wo"], out=h_mid, add=st["x"])
    st["h2"], rstd = K.rmsnorm_fwd(h_mid, st["w"]["ffn_norm"], d.eps)
    st["a"]["rstd_ffn"].copy_(rstd)


def stage_up_proj(K, d, st):
    _lin(K, st)(st["h2"], st["w"]["w13"], out=st["a"]["h13"])


def stage_swiglu(K, d, st):
    st["s"] = K.swiglu_packed_fwd(st["a"]["h13"])


def stage_down_resid(K, d, st):
    _lin(K, st)(st["s"], st["w"]["w2"], out=st["y"], add=st["a"]["h_mid"])


# ---- mixture-of-experts MLP (olmoe / qwen3moe variants): route -> dispatch + grouped up-projection -> SwiGLU ->
# grouped down-projection + weighted combine.  The routing decision and the row tables are saved context.
def stage_moe_route(K, d, st):
    a = st["a"]
    K.linear_fwd_bf16(st["h2"], st["w"]["w_router"], out=a["router_logits"])
    w, ids = K.moe_topk_softmax(a["router_logits"], d.topk, d.routing_mode)
    a["route_w"].copy_(w)
    a["route_ids"].copy_(ids)
    row_of, row_src, offp, tile_e, counts = K.moe_sort(ids, d.E)
    mp = row_src.shape[0]
    a["row_of"].copy_(row_of)
    a["row_src"][:mp].copy_(row_src)
    a["row_src"][mp:].fill_(-1)                 # rows past this round's content hold nothing
    a["offsets_pad"].copy_(offp)
    a["tile_expert"][:mp // 256].copy_(tile_e)
    a["tile_expert"][mp // 256:].fill_(-1)
    a["counts"].copy_(counts)


def stage_moe_up(K, d, st):
    a = st["a"]
    st["xp"] = K.moe_dispatch(st["h2"], a["row_src"])
    K.moe_grouped_mm(st["xp"], st["w"]["w13_experts"], a["tile_expert"], out=a["h13p"])


def stage_moe_act(K, d, st):
    st["sp"] = K.swiglu_packed_fwd(st["a"]["h13p"])


def stage_moe_down_combine(K, d, st):
    a = st["a"]
    yp = K.moe_grouped_mm(st["sp"], st["w"]["w2_experts"], a["tile_expert"])
    K.moe_combine(a["h_mid"], yp, a["route_w"], a["row_of"], out=st["y"])


# ---- the same MLP under expert parallelism: this rank holds E / ep experts and serves rows of every rank's tokens.
# The routing plan (which global token each local row holds, its weight, the padded expert ranges) is saved context;
# dispatch and combine are the fused kernels of ``parallel.ep.EpGroup``.
def _ep_group(st):
    g = st.get("ep")
    if g is None:
        raise RuntimeError("expert-parallel MoE stages need the group 'ep' (pass groups={'ep': EpGroup(...)})")
    return g


def ep_plan_from_context(a, d):
    from ...parallel.ep import EpPlan
    return EpPlan(ids=a["route_ids"], weights=a["route_w"], row_src=a["row_src"], row_slot=None, row_w=a["row_w"],
                  tile_expert=a["tile_expert"], offsets_pad=a["offsets_pad"], counts=a["counts"], rows_local=a["row_of"])


def stage_ep_route(K, d, st):
    a, g = st["a"], _ep_group(st)
    K.linear_fwd_bf16(st["h2"], st["w"]["w_router"], out=a["router_logits"])
    w, ids = K.moe_topk_softmax(a["router_logits"], d.topk, d.routing_mode)
    a["route_w"].copy_(w)
    a["route_ids"].copy_(ids)
    plan = g.plan(a["route_ids"], a["route_w"])
    for name in ("row_src", "row_w", "tile_expert", "offsets_pad"):
        a[name].copy_(getattr(plan, name))
    # the balance term is per rank and round, like the single-rank layer: counts of THIS rank's slots
    import torch
    flat = a["route_ids"].reshape(-1).long()
    a["counts"].copy_(torch.zeros(d.E, dtype=torch.int32, device=flat.device).scatter_add_(0, flat, torch.ones_like(flat, dtype=torch.int32)))
    st["plan"] = plan


def stage_ep_up(K, d, st):
    g, plan = _ep_group(st), st["plan"]
    st["xp"], st["h13p"] = g.dispatch_mm(st["h2"], st["w"]["w13_experts"], plan)
    st["a"]["row_of"].copy_(plan.rows_local)


def stage_ep_act(K, d, st):
    st["sp"] = K.swiglu_packed_fwd(st["h13p"])


def stage_ep_down_combine(K, d, st):
    g, a = _ep_group(st), st["a"]
    # the table stays where the rows are: the native grouped GEMM reads it on the device, the eager one copies it itself
    yp = K.moe_grouped_mm(st["sp"], st["w"]["w2_experts"], a["tile_expert"], out=g.rows_buffer() if g.lane == "p2p" else None)
    g.combine(yp, st["plan"], base=a["h_mid"], weighted=True, out=st["y"])


EP_ROUTE_FIELDS = ("router_logits", "route_w", "route_ids", "row_src", "row_w", "offsets_pad", "tile_expert", "counts")

MOE_ROUTE_FIELDS = ("router_logits", "route_w", "route_ids", "row_of", "row_src", "offsets_pad", "tile_expert", "counts")

STAGES_MOE = (
    ("attn_norm", stage_attn_norm, ("rstd_attn",)),
    ("qkv_rope", stage_qkv_rope, ("qkv",)),
    ("attn", stage_attn, ("lse", "attn_out")),
    ("resid1_norm2", stage_resid1_norm2, ("h_mid", "rstd_ffn")),
    ("moe_route", stage_moe_route, MOE_ROUTE_FIELDS),
    ("moe_up", stage_moe_up, ("h13p",)),
    ("moe_act", stage_moe_act, ()),
    ("moe_down_combine", stage_moe_down_combine, ()),
)

STAGES_EP = STAGES_MOE[:4] + (
    ("ep_route", stage_ep_route, EP_ROUTE_FIELDS),
    ("ep_up", stage_ep_up, ("row_of",)),
    ("ep_act", stage_ep_act, ()),
    ("ep_down_combine", stage_ep_down_combine, ()),
)

STAGES = (
    ("attn_norm", stage_attn_norm, ("rstd_attn",)),
    ("qkv_rope", stage_qkv_rope, ("qkv",)),
    ("attn", stage_attn, ("lse", "attn_out")),
    ("resid1_norm2", stage_resid1_norm2, ("h_mid", "rstd_ffn")),
    ("up_proj", stage_up_proj, ("h13",)),
    ("swiglu", stage_swiglu, ()),
    ("down_resid", stage_down_resid, ()),
)


def recompute_stages(stages=STAGES):
    """Stages up to and including the last one that emits saved context."""
    last = max(i for i, s in enumerate(stages) if s[2])
    return stages[:last + 1]


def context_rows(d, n):
    """Content-row trims of the context fields for an under-full round (token-axis aware)."""
    rows = {name: n for name in ("rstd_attn", "qkv", "attn_out", "h_mid", "rstd_ffn", "h13", "q_rstd", "k_rstd", "qk_pre",
                                 "router_logits", "route_w", "route_ids", "row_of")}
    return rows


class _Block(_Base):
    @property
    def stages(self):
        if getattr(self.dims, "moe", False):
            return STAGES_EP if self.dims.ep > 1 else STAGES_MOE
        return STAGES

    def ctx_views(self, buf, n):
        a = self.views(buf, self.lay.ctx, context_rows(self.dims, n))
        if n != self.dims.T:
            a = dict(a)
            a["lse"] = a["lse"][:, :n]
        return a

    def partial_views(self, buf, n):
        lay = self.lay.extra["Ap"]
        a = self.views(buf, lay, context_rows(self.dims, n))
        if n != self.dims.T:
            a = dict(a)
            a["lse"] = a["lse"][:, :n]
        return a

    def common(self, ctx, x_buf, w_buf):
        d = self.dims
        seg = self.segments(ctx)
        n = seg.n_tokens
        st = {"seg": seg, "n": n, "x": self.tview(x_buf, (d.T, d.d))[:n], "w": self.views(w_buf, self.lay.block_w),
              "fp8": self.hyper.get("linear_precision", "bf16") == "fp8"}
        if getattr(d, "ep", 1) > 1:
            if n != d.T:
                raise ValueError("expert-parallel blocks need full rounds (the peers pull exactly T rows from each rank)")
            st["ep"] = ctx.groups.get(ctx.task.comm_groups.get("ep", "ep"))
        return st


class BlockFwd(_Block):
    """(x, W) -> (y, A)"""

    def run(self, ctx):
        d = self.dims
        st = self.common(ctx, ctx.inputs[0], ctx.inputs[1])
        st["y"] = self.tview(ctx.outputs[0], (d.T, d.d))[:st["n"]]
        lvl = int(ctx.task.block_params.get("recompute_level", 0))
        if lvl == 0:
            st["a"] = self.ctx_views(ctx.outputs[1], st["n"])
        elif lvl == 1:
            # everything but h13 is saved (object Ap); h13 lives in scratch and is rebuilt before backward
            st["a"] = dict(self.partial_views(ctx.outputs[1], st["n"]))
            st["a"].update(self.scratch_ctx(st["n"], st["x"].device, only=("h13", "h13p")))
        else:
            st["a"] = self.scratch_ctx(st["n"], st["x"].device)      # context is dropped: recomputed before backward
        for _, fn, _ in self.stages:
            fn(self.K, d, st)

    def scratch_ctx(self, n, device, only=None):
        import torch
        from ...runtime.interop import _dtypes
        out = {}
        for f in self.lay.ctx.fields:
            if only is not None and f.name not in only:
                continue
            token_axis = f.name not in ("row_src", "offsets_pad", "tile_expert", "counts", "h13p")
            shape = (f.shape[0], n) if f.name == "lse" else ((n,) + tuple(f.shape[1:]) if token_axis else tuple(f.shape))
            out[f.name] = torch.empty(shape, dtype=_dtypes()[f.dtype], device=device)
        return out


class BlockRecompute(_Block):
    """(x, W) -> (A): the forward stages up to the last context-emitting one."""

    def run(self, ctx):
        st = self.common(ctx, ctx.inputs[0], ctx.inputs[1])
        st["a"] = self.ctx_views(ctx.outputs[0], st["n"])
        lvl = int(ctx.task.block_params.get("recompute_level", 2))
        if lvl == 1:
            # (x, W, Ap) -> A: copy the saved fields, rebuild h13 = rmsnorm(h_mid) @ w13
            saved = self.partial_views(ctx.inputs[2], st["n"])
            for name, t in saved.items():
                st["a"][name].copy_(t)
            st["h2"] = self.K.rmsnorm_apply(st["a"]["h_mid"], st["w"]["ffn_norm"], st["a"]["rstd_ffn"])
            (stage_moe_up if self.dims.moe else stage_up_proj)(self.K, self.dims, st)      # routing is saved context
            return
        for _, fn, _ in recompute_stages(self.stages):
            fn(self.K, self.dims, st)


class BlockBwd(_Block):
    """(dy, A, x, W[, dW]) -> (dx[, dW]); dW is created when it is an output, accumulated when mutated."""

    def run(self, ctx):
        import torch
        d, K = self.dims, self.K
        st = self.common(ctx, ctx.inputs[2], ctx.inputs[3])
        n, x, w, seg = st["n"], st["x"], st["w"], st["seg"]
        dy = self.tview(ctx.inputs[0], (d.T, d.d))[:n]
        a = self.ctx_views(ctx.inputs[1], n)
        dx = self.tview(ctx.outputs[0], (d.T, d.d))[:n]
        acc = not self.creating(ctx, "dW_")
        g = self.views(self.by_id(ctx, "dW_"), self.lay.block_dw)

        def wgrad(name, xin, dout):
            if name in g:                       # frozen fields have no gradient storage
                K.linear_wgrad_bf16(xin, dout, g[name], accumulate=acc)

        if d.moe and d.ep > 1:
            dh_mid = self.bwd_moe_ep(st["ep"], a, w, g, dy, acc, wgrad)
        else:
            dh_mid = (self.bwd_moe if d.moe else self.bwd_mlp)(a, w, g, dy, acc, wgrad)
        # ---- attention
        wgrad("wo", a["attn_out"], dh_mid)
        dattn = K.linear_dgrad_bf16(dh_mid, w["wo"])
        q, k, v = _qkv_views(d, a["qkv"], n)
        dqkv = torch.empty(n, d.qkv_dim, dtype=x.dtype, device=x.device)
        dq, dk, dv = _qkv_views(d, dqkv, n)
        K.flash_bwd(dattn.unflatten(1, (d.hq, d.hd)), q, k, v, a["attn_out"].unflatten(1, (d.hq, d.hd)), a["lse"],
                    seg.cu_seqlens, seg.max_len, dq=dq, dk=dk, dv=dv)
        del dattn
        K.rope_bwd(dq, seg.positions, d.theta)
        K.rope_bwd(dk, seg.positions, d.theta)
        if d.qk_norm:
            pre = a["qk_pre"]
            qp = _norm_rows(d, pre[:, :d.q_dim].unflatten(1, (d.hq, d.hd)))
            kp = _norm_rows(d, pre[:, d.q_dim:].unflatten(1, (d.hkv, d.hd)))
            dq.copy_(K.rmsnorm_bwd(_norm_rows(d, dq), qp, w["q_norm"], a["q_rstd"].reshape(-1), dw=g.get("q_norm"), accumulate=acc).view_as(dq))
            dk.copy_(K.rmsnorm_bwd(_norm_rows(d, dk), kp, w["k_norm"], a["k_rstd"].reshape(-1), dw=g.get("k_norm"), accumulate=acc).view_as(dk))
        h = K.rmsnorm_apply(x, w["attn_norm"], a["rstd_attn"])
        wgrad("w_qkv", h, dqkv)
        dh = K.linear_dgrad_bf16(dqkv, w["w_qkv"])
        K.rmsnorm_bwd(dh, x, w["attn_norm"], a["rstd_attn"], dx_add=dh_mid, dw=g.get("attn_norm"), accumulate=acc, out=dx)


    def bwd_mlp(self, a, w, g, dy, acc, wgrad):
        K = self.K
        h2 = K.rmsnorm_apply(a["h_mid"], w["ffn_norm"], a["rstd_ffn"])
        ds = K.linear_dgrad_bf16(dy, w["w2"])
        dh13, s = K.swiglu_packed_bwd(ds, a["h13"], with_s=True)      # one pass over h13 gives dh13 and the product s
        del ds
        wgrad("w2", s, dy)
        del s
        wgrad("w13", h2, dh13)
        dh2 = K.linear_dgrad_bf16(dh13, w["w13"])
        del dh13, h2
        return K.rmsnorm_bwd(dh2, a["h_mid"], w["ffn_norm"], a["rstd_ffn"], dx_add=dy, dw=g.get("ffn_norm"), accumulate=acc)

    def bwd_moe(self, a, w, g, dy, acc, wgrad):
        """Backward of route -> dispatch -> experts -> combine.  d(route_w)[t, k] = <dy[t], yp[row]> is taken as
        <dy W2^T, s> from the raw (unscaled) down-projection dgrad, then both are scaled by the route weight."""
        K, d = self.K, self.dims
        rw, row_of, tile_e, offp = a["route_w"], a["row_of"], a["tile_expert"], a["offsets_pad"]
        h2 = K.rmsnorm_apply(a["h_mid"], w["ffn_norm"], a["rstd_ffn"])
        xp = K.moe_dispatch(h2, a["row_src"])
        dyp = K.moe_dispatch(dy, a["row_src"])
        sp = K.swiglu_packed_fwd(a["h13p"])
        dsp = K.moe_grouped_mm(dyp, w["w2_experts"], tile_e, transpose_w=True)
        d_rw = K.moe_rowdot(dsp, sp, row_of)
        K.moe_scale_rows(dyp, rw, row_of)
        K.moe_scale_rows(dsp, rw, row_of)
        if "w2_experts" in g:
            K.moe_grouped_wgrad(sp, dyp, offp, g["w2_experts"], accumulate=acc)
        del sp, dyp
        dh13p = K.swiglu_packed_bwd(dsp, a["h13p"])
        del dsp
        if "w13_experts" in g:
            K.moe_grouped_wgrad(xp, dh13p, offp, g["w13_experts"], accumulate=acc)
        dxp = K.moe_grouped_mm(dh13p, w["w13_experts"], tile_e, transpose_w=True)
        del dh13p, xp
        dh2 = K.moe_dispatch_bwd(dxp, row_of)
        del dxp
        dlogits = K.moe_router_bwd(d_rw, rw, a["route_ids"], a["router_logits"], d.routing_mode)
        if d.aux_coef:
            K.moe_aux_lb_grad(a["router_logits"], a["counts"], dlogits, d.aux_coef, d.topk)
        dlog = dlogits.to(h2.dtype)
        wgrad("w_router", h2, dlog)
        dh2 = dh2 + K.linear_dgrad_bf16(dlog, w["w_router"])
        return K.rmsnorm_bwd(dh2, a["h_mid"], w["ffn_norm"], a["rstd_ffn"], dx_add=dy, dw=g.get("ffn_norm"), accumulate=acc)


    def bwd_moe_ep(self, grp, a, w, g, dy, acc, wgrad):
        """Expert-parallel backward: the rows of other ranks' tokens are pulled again (fused with the up-projection, which
        rebuilds h13p), dy is pulled fused with the down-projection's dgrad, and the owners of the tokens pull
        d(h2) and d(route_w) back in one combine."""
        K, d = self.K, self.dims
        plan = ep_plan_from_context(a, d)
        te = a["tile_expert"]
        h2 = K.rmsnorm_apply(a["h_mid"], w["ffn_norm"], a["rstd_ffn"])
        xp, h13p = grp.dispatch_mm(h2, w["w13_experts"], plan)
        sp = K.swiglu_packed_fwd(h13p)
        dyp, dsp = grp.dispatch_mm(dy, w["w2_experts"], plan, transpose_w=True)
        dscal = (dsp.float() * sp.float()).sum(-1)                       # <dy W2^T, s> per row, before scaling
        rw = plan.row_w.unsqueeze(-1)
        dsp = (dsp.float() * rw).to(dsp.dtype)
        dyp = (dyp.float() * rw).to(dyp.dtype)
        if "w2_experts" in g:
            K.moe_grouped_wgrad(sp, dyp, a["offsets_pad"], g["w2_experts"], accumulate=acc)
        del sp, dyp
        dh13p = K.swiglu_packed_bwd(dsp, h13p)
        del dsp, h13p
        if "w13_experts" in g:
            K.moe_grouped_wgrad(xp, dh13p, a["offsets_pad"], g["w13_experts"], accumulate=acc)
        dxp = K.moe_grouped_mm(dh13p, w["w13_experts"], te, out=grp.rows_buffer() if grp.lane == "p2p" else None, transpose_w=True)
        del dh13p, xp
        dh2, d_rw = grp.combine(dxp, plan, base=None, weighted=False, scal=dscal)
        dlogits = K.moe_router_bwd(d_rw, a["route_w"], a["route_ids"], a["router_logits"], d.routing_mode)
        if d.aux_coef:
            K.moe_aux_lb_grad(a["router_logits"], a["counts"], dlogits, d.aux_coef, d.topk)
        dlog = dlogits.to(h2.dtype)
        wgrad("w_router", h2, dlog)
        dh2 = dh2 + K.linear_dgrad_bf16(dlog, w["w_router"])
        return K.rmsnorm_bwd(dh2, a["h_mid"], w["ffn_norm"], a["rstd_ffn"], dx_add=dy, dw=g.get("ffn_norm"), accumulate=acc)


def build_llama3_resolver(dims, hyper: Mapping[str, Any] | None, kernels, device, layouts=None, policy=None):
    from .model import family_layouts
    from ...blocks.layouts import DTypePolicy
    hyper = dict(hyper or {})
    lay = layouts or family_layouts(dims, policy or DTypePolicy.from_dict(hyper.get("dtype_policy", "bf16")),
                                    hyper.get("optimizer", "adamw"))
    table = common_executables(dims, lay, kernels, device, hyper)
    if getattr(dims, "ep", 1) > 1:
        # every rank sees different tokens: gradients of everything but the (rank-local) experts are summed over the group
        from ..tp_mlp.blocks import ReplicatedGradSum
        table["optimizer_block"] = ReplicatedGradSum(table["optimizer_block"], lay.block_dw, None, "ep", skip=("w13_experts", "w2_experts"))
        table["optimizer_embed"] = ReplicatedGradSum(table["optimizer_embed"], lay.embed_dw, None, "ep")
        table["optimizer_head"] = ReplicatedGradSum(table["optimizer_head"], lay.head_dw, None, "ep")
    table.update({
        "block_fwd": BlockFwd(dims, lay, kernels, device, hyper),
        "block_recompute": BlockRecompute(dims, lay, kernels, device, hyper),
        "block_bwd": BlockBwd(dims, lay, kernels, device, hyper),
    })

    def resolver(task):
        try:
            return table[task.compute_block_key]
        except KeyError:
            raise KeyError(f"llama3: no executable for compute key {task.compute_block_key!r} (task {task.id})") from None
    resolver.table = table
    return resolver
