"""Executables of the tensor + sequence parallel llama block.

Shapes on one rank (``T`` rows per round, ``Ts = T / tp`` of them its own, local heads / FFN columns):

    x, y, h_mid            (Ts, d)          the residual stream, row-sharded
    qkv, attn_out, h13     (T, local)       every row of this rank's heads / columns

Forward:   rmsnorm -> [all-gather -> qkv GEMM] -> rope, attention -> [wo GEMM -> reduce-scatter (+x)] -> rmsnorm
           -> [all-gather -> w13 GEMM] -> SwiGLU -> [w2 GEMM -> reduce-scatter (+h_mid)]
Backward:  the transposes of the four bracketed kernels in reverse; weight gradients of the column-parallel matrices
           contract over all T rows, for which the gathered operand of the fused kernel (or one plain all-gather of
           the re-applied norm) is used; norm-weight gradients are partial sums over this rank's rows and are summed
           over the group by the optimizer wrapper.
Reference role: ``src/dataflow_training/model_families/tp_mlp/`` (MLP-only sharding, NCCL all-reduce).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping

from ...blocks.base_blocks import _Base, common_executables
from ...data.segments import make_segments
from ..llama3.blocks import _qkv_views


def _group(ctx, key: str = "tp"):
    g = ctx.groups.get(ctx.task.comm_groups.get(key, key))
    if g is None:
        raise RuntimeError(f"task {ctx.task.id} needs the group {key!r} (pass groups={{{key!r}: ...}})")
    return g


class _TpBlock(_Base):
    def rows(self, ctx):
        seg = self.segments(ctx)
        if seg.n_tokens != self.dims.T:
            raise ValueError("tensor-parallel blocks need full rounds (every rank holds exactly T / tp rows)")
        return seg

    def ctx_views(self, buf):
        return self.views(buf, self.lay.ctx)

    def scratch_ctx(self, device, only=None):
        import torch
        from ...runtime.interop import _dtypes
        return {f.name: torch.empty(tuple(f.shape), dtype=_dtypes()[f.dtype], device=device)
                for f in self.lay.ctx.fields if only is None or f.name in only}

    # -- forward pieces
    def attention_half(self, g, K, d, seg, x, w, a):
        h, rstd = K.rmsnorm_fwd(x, w["attn_norm"], d.eps)
        a["rstd_attn"].copy_(rstd)
        g.ag_gemm(h, w["w_qkv"], out=a["qkv"])
        q, k, v = _qkv_views(d, a["qkv"], d.T)
        K.rope_fwd(q, seg.positions, d.theta)
        K.rope_fwd(k, seg.positions, d.theta)
        _, lse = K.flash_fwd(q, k, v, seg.cu_seqlens, seg.max_len, out=a["attn_out"].unflatten(1, (d.hq, d.hd)))
        a["lse"].copy_(lse)
        g.gemm_rs(a["attn_out"], w["wo"], out=a["h_mid"], addend=x)

    def up_projection(self, g, K, d, w, a):
        h2, rstd = K.rmsnorm_fwd(a["h_mid"], w["ffn_norm"], d.eps)
        a["rstd_ffn"].copy_(rstd)
        g.ag_gemm(h2, w["w13"], out=a["h13"])


class TpBlockFwd(_TpBlock):
    """(x, W) -> (y, A)"""

    def run(self, ctx):
        d, K, g = self.dims, self.K, _group(ctx)
        seg = self.rows(ctx)
        x = self.tview(ctx.inputs[0], (d.Ts, d.d))
        w = self.views(ctx.inputs[1], self.lay.block_w)
        y = self.tview(ctx.outputs[0], (d.Ts, d.d))
        lvl = int(ctx.task.block_params.get("recompute_level", 0))
        if lvl == 0:
            a = self.ctx_views(ctx.outputs[1])
        elif lvl == 1:
            a = dict(self.views(ctx.outputs[1], self.lay.extra["Ap"]))
            a.update(self.scratch_ctx(x.device, only=("h13",)))
        else:
            a = self.scratch_ctx(x.device)
        self.attention_half(g, K, d, seg, x, w, a)
        self.up_projection(g, K, d, w, a)
        s = K.swiglu_packed_fwd(a["h13"])
        g.gemm_rs(s, w["w2"], out=y, addend=a["h_mid"])


class TpBlockRecompute(_TpBlock):
    """(x, W[, Ap]) -> (A)"""

    def run(self, ctx):
        d, K, g = self.dims, self.K, _group(ctx)
        seg = self.rows(ctx)
        x = self.tview(ctx.inputs[0], (d.Ts, d.d))
        w = self.views(ctx.inputs[1], self.lay.block_w)
        a = self.ctx_views(ctx.outputs[0])
        if int(ctx.task.block_params.get("recompute_level", 2)) == 1:
            for name, t in self.views(ctx.inputs[2], self.lay.extra["Ap"]).items():
                a[name].copy_(t)
            h2 = K.rmsnorm_apply(a["h_mid"], w["ffn_norm"], a["rstd_ffn"])
            g.ag_gemm(h2, w["w13"], out=a["h13"])
            return
        self.attention_half(g, K, d, seg, x, w, a)
        self.up_projection(g, K, d, w, a)


class TpBlockBwd(_TpBlock):
    """(dy, A, x, W[, dW]) -> (dx[, dW])"""

    def run(self, ctx):
        import torch
        d, K, g = self.dims, self.K, _group(ctx)
        seg = self.rows(ctx)
        dy = self.tview(ctx.inputs[0], (d.Ts, d.d))
        a = self.ctx_views(ctx.inputs[1])
        x = self.tview(ctx.inputs[2], (d.Ts, d.d))
        w = self.views(ctx.inputs[3], self.lay.block_w)
        dx = self.tview(ctx.outputs[0], (d.Ts, d.d))
        acc = not self.creating(ctx, "dW_")
        gr = self.views(self.by_id(ctx, "dW_"), self.lay.block_dw)

        def wgrad(name, xin, dout):
            if name in gr:
                K.linear_wgrad_bf16(xin, dout, gr[name], accumulate=acc)

        # ---- MLP
        ds = g.ag_gemm(dy, w["w2"], w_is_kn=False)                      # dy (all rows) x W2^T, gather fused
        dh13, s = K.swiglu_packed_bwd(ds, a["h13"], with_s=True)        # one pass over h13: dh13 and the forward product
        del ds
        wgrad("w2", s, g.last_gathered(d.Ts, d.d))
        del s
        h2 = K.rmsnorm_apply(a["h_mid"], w["ffn_norm"], a["rstd_ffn"])
        wgrad("w13", g.all_gather(h2), dh13)
        del h2
        dh2 = g.gemm_rs(dh13, w["w13"], w_is_kn=False)                  # dh13 x W13^T, reduce-scatter fused
        del dh13
        dh_mid = K.rmsnorm_bwd(dh2, a["h_mid"], w["ffn_norm"], a["rstd_ffn"], dx_add=dy, dw=gr.get("ffn_norm"), accumulate=acc)
        # ---- attention
        dattn = g.ag_gemm(dh_mid, w["wo"], w_is_kn=False)
        wgrad("wo", a["attn_out"], g.last_gathered(d.Ts, d.d))
        q, k, v = _qkv_views(d, a["qkv"], d.T)
        dqkv = torch.empty(d.T, d.qkv_dim, dtype=x.dtype, device=x.device)
        dq, dk, dv = _qkv_views(d, dqkv, d.T)
        K.flash_bwd(dattn.unflatten(1, (d.hq, d.hd)), q, k, v, a["attn_out"].unflatten(1, (d.hq, d.hd)), a["lse"],
                    seg.cu_seqlens, seg.max_len, dq=dq, dk=dk, dv=dv)
        del dattn
        K.rope_bwd(dq, seg.positions, d.theta)
        K.rope_bwd(dk, seg.positions, d.theta)
        h = K.rmsnorm_apply(x, w["attn_norm"], a["rstd_attn"])
        wgrad("w_qkv", g.all_gather(h), dqkv)
        del h
        dh = g.gemm_rs(dqkv, w["w_qkv"], w_is_kn=False)
        K.rmsnorm_bwd(dh, x, w["attn_norm"], a["rstd_attn"], dx_add=dh_mid, dw=gr.get("attn_norm"), accumulate=acc, out=dx)


class VocabParallelHeadLoss(_Base):
    """(y, targets, W_head) -> (dy, loss[, dW_head]) with the vocabulary columns of the output projection split over the
    group: the normalised rows are all-gathered, every rank computes the logits of its columns, and the softmax statistics
    (row maximum, sum of exponentials, the target's logit) are exchanged — two sums and one maximum of ``T`` floats per
    chunk — so neither the full logits nor the full matrix exist on any rank.  The gradient of the gathered rows is summed
    over the group and every rank keeps its rows.  Written with library collectives around the GEMM ops (no fused kernel)."""

    def run(self, ctx):
        import torch
        d, K, g = self.dims, self.K, _group(ctx)
        Ts, Vl = d.Ts, d.vocab_local
        y = self.tview(ctx.inputs[0], (Ts, d.d))
        tgt = self.tview(ctx.inputs[1], (Ts,), "int32")
        w = self.views(ctx.inputs[2], self.lay.head_w)
        dy = self.tview(ctx.outputs[0], (Ts, d.d))
        loss = self.tview(ctx.outputs[1], (1,), "fp32")
        create = self.creating(ctx, "dW_head")
        dw = self.views(self.by_id(ctx, "dW_head"), self.lay.head_dw)
        total_rows = float(ctx.run_args.get("valid_rows", d.T))
        xn, rstd = K.rmsnorm_fwd(y, w["final_norm"], d.eps)
        xg = g.all_gather(xn)                                               # (T, d): every row, this rank's columns follow
        tg = g.all_gather(tgt.reshape(-1, 1).contiguous()).reshape(-1).long()
        v0 = g.rank * Vl
        dxg = torch.empty(d.T, d.d, dtype=torch.float32, device=y.device)
        total = torch.zeros((), dtype=torch.float32, device=y.device)
        first = True
        for lo in range(0, d.T, max(int(d.head_chunk), 1)):
            hi = min(lo + max(int(d.head_chunk), 1), d.T)
            logits = K.linear_fwd_bf16(xg[lo:hi], w["w_head"]).float()      # (rows, Vl)
            m = g.all_reduce(logits.max(-1).values.contiguous(), op="max")
            e = torch.exp(logits - m[:, None])
            se = g.all_reduce(e.sum(-1))
            t = tg[lo:hi]
            valid = (t >= 0).float()
            mine = (t >= v0) & (t < v0 + Vl)
            idx = (t - v0).clamp(0, Vl - 1)[:, None]
            tl = g.all_reduce(torch.where(mine, logits.gather(1, idx)[:, 0], torch.zeros_like(m)))
            total += (((m + torch.log(se)) - tl) * valid).sum() / total_rows
            p = e / se[:, None]
            p.scatter_add_(1, idx, -mine.float()[:, None])
            dl = (p * (valid / total_rows)[:, None]).to(xg.dtype)
            K.linear_wgrad_bf16(xg[lo:hi], dl, dw["w_head"], accumulate=not (create and first))
            dxg[lo:hi] = K.linear_dgrad_bf16(dl, w["w_head"]).float()
            first = False
        g.all_reduce(dxg)
        K.rmsnorm_bwd(dxg[g.rank * Ts:(g.rank + 1) * Ts].to(y.dtype).contiguous(), y, w["final_norm"], rstd, dw=dw["final_norm"],
                      accumulate=not create, out=dy)
        loss.copy_((total / g.world).reshape(1), non_blocking=True)        # every rank holds the round's loss: the job sums ranks


class _ShardRows:
    """Row-sharded executables see one segment of ``Ts`` rows (they need the row count, not the sequence structure)."""

    def segments(self, ctx):
        seg = getattr(self, "_seg", None)
        if seg is None:
            seg = self._seg = make_segments([0, self.dims.T], self.device)
        return seg


class ReplicatedGradSum:
    """Wraps an optimizer executable: sums the gradients of parameters every rank holds in full over the group first.
    ``fields``: names inside the packed gradient object, or ``None`` for all of them."""

    def __init__(self, inner, layout_of_grad, fields, group: str = "tp", skip=()):
        self.inner, self.layout_of_grad, self.fields, self.group, self.skip = inner, layout_of_grad, fields, group, tuple(skip)

    def __getattr__(self, name):
        # wrappers stack (sum over the tensor-parallel group, then over the data-parallel replicas): the layout helpers and the
        # device of the innermost executable show through
        return getattr(self.__dict__["inner"], name)

    def launch(self, ctx):
        inner = self.inner
        if inner.device is None:
            return self.run(ctx)
        import torch
        from ...runtime.interop import external_stream
        with torch.cuda.stream(external_stream(ctx.stream, inner.device)):
            self.run(ctx)

    def run(self, ctx):
        g = _group(ctx, self.group)
        views = self.inner.views(ctx.inputs[1], self.layout_of_grad)
        for name, t in views.items():
            if (self.fields is None or name in self.fields) and name not in self.skip:
                g.all_reduce(t)
        self.inner.run(ctx)


def build_tp_resolver(dims, hyper: Mapping[str, Any] | None, kernels, device, layouts=None, policy=None):
    from ...blocks.layouts import DTypePolicy
    from ..llama3.model import family_layouts
    hyper = dict(hyper or {})
    lay = layouts or family_layouts(dims, policy or DTypePolicy.from_dict(hyper.get("dtype_policy", "bf16")), hyper.get("optimizer", "adamw"))
    sd = dataclasses.replace(dims, T=dims.Ts, tp=1, head_chunk=min(dims.head_chunk, dims.Ts))
    table = {}
    for key, exe in common_executables(sd, lay, kernels, device, hyper).items():
        cls = type(exe)
        table[key] = type("Shard" + cls.__name__, (_ShardRows, cls), {})(sd, lay, kernels, device, hyper)
    table["optimizer_block"] = ReplicatedGradSum(table["optimizer_block"], lay.block_dw, ("attn_norm", "ffn_norm"))
    table["optimizer_embed"] = ReplicatedGradSum(table["optimizer_embed"], lay.embed_dw, None)
    table["optimizer_head"] = ReplicatedGradSum(table["optimizer_head"], lay.head_dw, None)
    if int(getattr(dims, "head_shard", 1)) > 1:
        table["head_loss"] = VocabParallelHeadLoss(dims, lay, kernels, device, hyper)
        table["optimizer_head"] = ReplicatedGradSum(table["optimizer_head"].inner, lay.head_dw, ("final_norm",))
    table.update({"block_fwd": TpBlockFwd(dims, lay, kernels, device, hyper),
                  "block_recompute": TpBlockRecompute(dims, lay, kernels, device, hyper),
                  "block_bwd": TpBlockBwd(dims, lay, kernels, device, hyper)})

    def resolver(task):
        try:
            return table[task.compute_block_key]
        except KeyError:
            raise KeyError(f"tp_mlp: no executable for compute key {task.compute_block_key!r} (task {task.id})") from None
    resolver.table = table
    return resolver
