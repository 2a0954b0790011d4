"""gpt2 block executables (staged forward, derived recompute, backward with bias gradients).
Structure parity: reference ``src/dataflow_training/model_families/gpt2/blocks.py:51-426``."""
from __future__ import annotations

from typing import Any, Mapping

from ...blocks.base_blocks import HeadLoss, _Base, common_executables


def _split(d, qkv):
    q = qkv[:, :d.d].unflatten(1, (d.hq, d.hd))
    k = qkv[:, d.d:2 * d.d].unflatten(1, (d.hq, d.hd))
    v = qkv[:, 2 * d.d:].unflatten(1, (d.hq, d.hd))
    return q, k, v


def stage_ln1(K, d, st):
    w = st["w"]
    st["h"], mean, rstd = K.layernorm_fwd(st["x"], w["ln1_w"], w.get("ln1_b"), d.eps)
    st["a"]["mean1"].copy_(mean)
    st["a"]["rstd1"].copy_(rstd)


def stage_qkv(K, d, st):
    K.linear_fwd_bf16(st["h"], st["w"]["c_attn_w"], out=st["a"]["qkv"], bias=st["w"].get("c_attn_b"))


def stage_attn(K, d, st):
    q, k, v = _split(d, st["a"]["qkv"])
    out = st["a"]["attn_out"].unflatten(1, (d.hq, d.hd))
    _, lse = K.flash_fwd(q, k, v, st["seg"].cu_seqlens, st["seg"].max_len, out=out)
    st["a"]["lse"].copy_(lse)


def stage_proj_ln2(K, d, st):
    w, a = st["w"], st["a"]
    K.linear_fwd_bf16(a["attn_out"], w["attn_proj_w"], out=a["h_mid"], add=st["x"], bias=w.get("attn_proj_b"))
    st["h2"], mean, rstd = K.layernorm_fwd(a["h_mid"], w["ln2_w"], w.get("ln2_b"), d.eps)
    a["mean2"].copy_(mean)
    a["rstd2"].copy_(rstd)


def stage_fc(K, d, st):
    K.linear_fwd_bf16(st["h2"], st["w"]["fc_w"], out=st["a"]["fc"], bias=st["w"].get("fc_b"))


def stage_gelu(K, d, st):
    st["g"] = K.gelu_fwd_out(st["a"]["fc"])


def stage_out(K, d, st):
    K.linear_fwd_bf16(st["g"], st["w"]["mlp_proj_w"], out=st["y"], add=st["a"]["h_mid"], bias=st["w"].get("mlp_proj_b"))


STAGES = (
    ("ln1", stage_ln1, ("mean1", "rstd1")),
    ("qkv", stage_qkv, ("qkv",)),
    ("attn", stage_attn, ("lse", "attn_out")),
    ("proj_ln2", stage_proj_ln2, ("h_mid", "mean2", "rstd2")),
    ("fc", stage_fc, ("fc",)),
    ("gelu", stage_gelu, ()),
    ("out", stage_out, ()),
)

_TOKEN_FIELDS = ("mean1", "rstd1", "qkv", "attn_out", "h_mid", "mean2", "rstd2", "fc")


class _Block(_Base):
    stages = STAGES

    def _views(self, buf, layout, n):
        a = self.views(buf, layout, {k: n for k in _TOKEN_FIELDS})
        if n != self.dims.T:
            a = dict(a)
            a["lse"] = a["lse"][:, :n]
        return a

    def ctx_views(self, buf, n):
        return self._views(buf, self.lay.ctx, n)

    def partial_views(self, buf, n):
        return self._views(buf, self.lay.extra["Ap"], n)

    def scratch_ctx(self, n, device, only=None):
        import torch
        from ...runtime.interop import _dtypes
        out = {}
        for f in self.lay.ctx.fields:
            if only is not None and f.name not in only:
                continue
            shape = (f.shape[0], n) if f.name == "lse" else (n,) + tuple(f.shape[1:])
            out[f.name] = torch.empty(shape, dtype=_dtypes()[f.dtype], device=device)
        return out

    def common(self, ctx, x_buf, w_buf):
        d = self.dims
        seg = self.segments(ctx)
        n = seg.n_tokens
        return {"seg": seg, "n": n, "x": self.tview(x_buf, (d.T, d.d))[:n], "w": self.views(w_buf, self.lay.block_w)}


class BlockFwd(_Block):
    def run(self, ctx):
        d = self.dims
        st = self.common(ctx, ctx.inputs[0], ctx.inputs[1])
        st["y"] = self.tview(ctx.outputs[0], (d.T, d.d))[:st["n"]]
        lvl = int(ctx.task.block_params.get("recompute_level", 0))
        if lvl == 0:
            st["a"] = self.ctx_views(ctx.outputs[1], st["n"])
        elif lvl == 1:
            st["a"] = dict(self.partial_views(ctx.outputs[1], st["n"]))
            st["a"].update(self.scratch_ctx(st["n"], st["x"].device, only=("fc",)))
        else:
            st["a"] = self.scratch_ctx(st["n"], st["x"].device)
        for _, fn, _ in self.stages:
            fn(self.K, d, st)


class BlockRecompute(_Block):
    def run(self, ctx):
        st = self.common(ctx, ctx.inputs[0], ctx.inputs[1])
        st["a"] = self.ctx_views(ctx.outputs[0], st["n"])
        lvl = int(ctx.task.block_params.get("recompute_level", 2))
        if lvl == 1:
            for name, t in self.partial_views(ctx.inputs[2], st["n"]).items():
                st["a"][name].copy_(t)
            w, a = st["w"], st["a"]
            st["h2"] = self.K.layernorm_apply(a["h_mid"], w["ln2_w"], w.get("ln2_b"), a["mean2"], a["rstd2"])
            stage_fc(self.K, self.dims, st)
            return
        for _, fn, _ in self.stages[:5]:
            fn(self.K, self.dims, st)


class BlockBwd(_Block):
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
            if name in g:
                K.linear_wgrad_bf16(xin, dout, g[name], accumulate=acc)

        def bgrad(name, dout):
            if name in g:
                K.bias_grad(dout, g[name], accumulate=acc)

        h2 = K.layernorm_apply(a["h_mid"], w["ln2_w"], w.get("ln2_b"), a["mean2"], a["rstd2"])
        gact = K.gelu_fwd_out(a["fc"])
        wgrad("mlp_proj_w", gact, dy)
        bgrad("mlp_proj_b", dy)
        dg = K.linear_dgrad_bf16(dy, w["mlp_proj_w"])
        dfc = K.gelu_bwd(dg, a["fc"])
        wgrad("fc_w", h2, dfc)
        bgrad("fc_b", dfc)
        dh2 = K.linear_dgrad_bf16(dfc, w["fc_w"])
        dh_mid = K.layernorm_bwd(dh2, a["h_mid"], w["ln2_w"], a["mean2"], a["rstd2"], dx_add=dy, dw=g.get("ln2_w"),
                                 db=g.get("ln2_b"), accumulate=acc)
        wgrad("attn_proj_w", a["attn_out"], dh_mid)
        bgrad("attn_proj_b", dh_mid)
        dattn = K.linear_dgrad_bf16(dh_mid, w["attn_proj_w"])
        q, k, v = _split(d, a["qkv"])
        dqkv = torch.empty(n, 3 * d.d, dtype=x.dtype, device=x.device)
        dq, dk, dv = _split(d, dqkv)
        K.flash_bwd(dattn.unflatten(1, (d.hq, d.hd)), q, k, v, a["attn_out"].unflatten(1, (d.hq, d.hd)), a["lse"],
                    seg.cu_seqlens, seg.max_len, dq=dq, dk=dk, dv=dv)
        h = K.layernorm_apply(x, w["ln1_w"], w.get("ln1_b"), a["mean1"], a["rstd1"])
        wgrad("c_attn_w", h, dqkv)
        bgrad("c_attn_b", dqkv)
        dh = K.linear_dgrad_bf16(dqkv, w["c_attn_w"])
        K.layernorm_bwd(dh, x, w["ln1_w"], a["mean1"], a["rstd1"], dx_add=dh_mid, dw=g.get("ln1_w"), db=g.get("ln1_b"),
                        accumulate=acc, out=dx)


class Gpt2HeadLoss(HeadLoss):
    norm = "layer"


def build_gpt2_resolver(dims, hyper: Mapping[str, Any] | None, kernels, device, layouts=None, policy=None):
    from ...blocks.layouts import DTypePolicy
    from .model import family_layouts
    hyper = dict(hyper or {})
    lay = layouts or family_layouts(dims, policy or DTypePolicy.from_dict(hyper.get("dtype_policy", "bf16")),
                                    hyper.get("optimizer", "adamw"))
    table = common_executables(dims, lay, kernels, device, hyper)
    table.update({"head_loss": Gpt2HeadLoss(dims, lay, kernels, device, hyper),
                  "block_fwd": BlockFwd(dims, lay, kernels, device, hyper),
                  "block_recompute": BlockRecompute(dims, lay, kernels, device, hyper),
                  "block_bwd": BlockBwd(dims, lay, kernels, device, hyper)})

    def resolver(task):
        try:
            return table[task.compute_block_key]
        except KeyError:
            raise KeyError(f"gpt2: no executable for compute key {task.compute_block_key!r} (task {task.id})") from None
    resolver.table = table
    return resolver
