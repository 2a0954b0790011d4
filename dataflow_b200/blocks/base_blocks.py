"""Executables shared by every family: round prologue, embedding forward/backward,
chunked head + loss, per-object optimizer step.

An executable's ``launch(ctx)`` only enqueues work on the engine's compute
stream; buffers are addressed positionally (fwd ``(x, W) -> (y, A)``, bwd
``(dy, A, x, W[, dW]) -> (dx[, dW])``, head ``(y, targets, W_head) -> (dy, loss[, dW_head])``,
optimizer ``(W, dW, O)``) and whether a gradient is *created* or *accumulated*
comes from the task (``dW`` in outputs vs in mutates), never from the round
number.  Contract parity: reference ``src/dataflow_training/blocks/base_blocks.py:38-728``,
``docs/program_contract.md:73-81``.
"""
from __future__ import annotations

import fnmatch

import math
from typing import Any, Mapping

from ..data.segments import resolve_segments
from .optim import lr_at


class _Base:
    """Layout helpers + stream scoping.  ``device`` is a CUDA ordinal or ``None`` for host tensors."""

    def __init__(self, dims, layouts, kernels, device, hyper: Mapping[str, Any] | None = None):
        self.dims = dims
        self.lay = layouts
        self.K = kernels
        self.device = device
        self.hyper = dict(hyper or {})

    def launch(self, ctx) -> None:
        if self.device is None:
            return self.run(ctx)
        import torch
        from ..runtime.interop import external_stream
        with torch.cuda.stream(external_stream(ctx.stream, self.device)):
            pending = ctx.run_values.get("_ready")
            if pending:
                # inputs produced on another stream (asynchronous gathers / reduce-scatters): wait on-stream
                # The stall is timed on the device: an event in front of the wait fires when the compute stream gets there,
                # one behind it when the transfer's event has fired too; their distance is communication the step could
                # not hide (``exposed_comm_us`` of the run's statistics).
                cur = torch.cuda.current_stream()
                evs = [ev for ev in (pending.pop(b.object_id, None) for b in ctx.inputs) if ev is not None]
                if evs:
                    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    t0.record(cur)
                    for ev in evs:
                        cur.wait_event(ev)
                    t1.record(cur)
                    ctx.run_values.setdefault("_comm_waits", []).append((t0, t1))
            self.run(ctx)

    def run(self, ctx) -> None:      # pragma: no cover - abstract
        raise NotImplementedError

    # -- views
    def views(self, buf, layout, rows=None):
        dev = self.device if buf.location == "fast" else None
        return layout.views(buf, dev, rows)

    def tview(self, buf, shape, dtype=None):
        from ..runtime.interop import torch_view
        dtype = dtype or getattr(self.dims, "act", "bf16")       # activations follow the family's activation dtype
        return torch_view(buf, shape, dtype, 0, self.device if buf.location == "fast" else None)

    def by_id(self, ctx, prefix: str):
        for b in ctx.inputs:
            if b.object_id.startswith(prefix):
                return b
        for b in ctx.outputs:
            if b.object_id.startswith(prefix):
                return b
        return None

    def segments(self, ctx):
        r = int(ctx.task.block_params.get("round", 0))
        return resolve_segments(ctx, r, self.dims.T, self.dims.seq_len, self.device)

    def creating(self, ctx, prefix: str) -> bool:
        """True when the gradient object ``prefix*`` is an output of this task (round 0)."""
        return any(o.object_id.startswith(prefix) for o in ctx.outputs)


class RoundPrologue(_Base):
    """Publishes the round index as a 4-byte device object (and nothing else)."""

    def run(self, ctx):
        out = self.tview(ctx.outputs[0], (1,), "int32")
        out.fill_(int(ctx.task.block_params.get("round", 0)))


class EmbedFwd(_Base):
    def run(self, ctx):
        seg = self.segments(ctx)
        n = seg.n_tokens
        tok = self.tview(ctx.inputs[0], (self.dims.T,), "int32")[:n]
        w = self.views(ctx.inputs[1], self.lay.embed_w)
        y = self.tview(ctx.outputs[0], (self.dims.T, self.dims.d))[:n]
        pos_table = w.get("wpe")
        self.K.embed_fwd(tok, w["wte"], y, seg.positions if pos_table is not None else None, pos_table)


class EmbedBwd(_Base):
    def run(self, ctx):
        seg = self.segments(ctx)
        n = seg.n_tokens
        dy = self.tview(ctx.inputs[0], (self.dims.T, self.dims.d))[:n]
        tok = self.tview(ctx.inputs[1], (self.dims.T,), "int32")[:n]
        create = self.creating(ctx, "dW_embed")
        dwb = self.by_id(ctx, "dW_embed")
        dw = self.views(dwb, self.lay.embed_dw)
        self.K.embed_bwd_accum(tok, dy, dw["wte"], accumulate=not create)
        if "wpe" in dw:
            self.K.embed_bwd_accum(seg.positions, dy, dw["wpe"], accumulate=not create)


class HeadLoss(_Base):
    """Final norm → head GEMM → fused CE → dW_head → dgrad → norm backward, token-chunked so
    the (tokens x vocab) logits never exist at once."""

    norm = "rms"

    def run(self, ctx):
        import torch
        d, K = self.dims, self.K
        seg = self.segments(ctx)
        n = seg.n_tokens
        y = self.tview(ctx.inputs[0], (d.T, d.d))[:n]
        tgt = self.tview(ctx.inputs[1], (d.T,), "int32")[:n]
        w = self.views(ctx.inputs[2], self.lay.head_w)
        dy = self.tview(ctx.outputs[0], (d.T, d.d))[:n]
        loss = self.tview(ctx.outputs[1], (1,), "fp32")
        create = self.creating(ctx, "dW_head")
        dw = self.views(self.by_id(ctx, "dW_head"), self.lay.head_dw)
        tied = "w_head" not in w
        if tied:
            w_head_t = self.views(self.by_id(ctx, "W_embed"), self.lay.embed_w)["wte"]      # (vocab, d)
            dwe_all = self.views(self.by_id(ctx, "dW_embed"), self.lay.embed_dw)
            dwe = dwe_all["wte"]
            create_e = self.creating(ctx, "dW_embed")
            if create_e:
                # this task creates the shared gradient object: fields it does not write start at zero
                for name, t in dwe_all.items():
                    if name != "wte":
                        t.zero_()
        total_rows = float(ctx.run_args.get("valid_rows", n))
        dev = y.device
        loss_dev = torch.zeros(1, dtype=torch.float32, device=dev)
        first = True
        for lo in range(0, n, d.head_chunk):
            hi = min(lo + d.head_chunk, n)
            yc = y[lo:hi]
            if self.norm == "rms":
                xn, rstd = K.rmsnorm_fwd(yc, w["final_norm"], d.eps)
            else:
                xn, mean, rstd = K.layernorm_fwd(yc, w["final_norm"], w.get("final_norm_b"), d.eps)
            if tied:
                logits = K.linear_dgrad_bf16(xn, w_head_t)                 # xn @ wte^T
            else:
                logits = K.linear_fwd_bf16(xn, w["w_head"])
            K.ce_loss_fwd_bwd(logits, tgt[lo:hi], total_rows, loss_dev, accumulate=not first)
            acc = not (create and first)
            if tied:
                # d(wte) += dlogits^T @ xn
                K.linear_wgrad_bf16(logits, xn, dwe, accumulate=not (create_e and first))
                dxn = K.linear_fwd_bf16(logits, w_head_t)
            else:
                K.linear_wgrad_bf16(xn, logits, dw["w_head"], accumulate=acc)
                dxn = K.linear_dgrad_bf16(logits, w["w_head"])
            if self.norm == "rms":
                K.rmsnorm_bwd(dxn, yc, w["final_norm"], rstd, dw=dw["final_norm"], accumulate=acc, out=dy[lo:hi])
            else:
                K.layernorm_bwd(dxn, yc, w["final_norm"], mean, rstd, dw=dw["final_norm"], db=dw.get("final_norm_b"),
                                accumulate=acc, out=dy[lo:hi])
            first = False
        loss.copy_(loss_dev, non_blocking=True)


class OptimizerStep(_Base):
    """Per-field optimizer update over one packed (W, dW, O) triple.

    ``block_params["target"]`` picks the layouts (block / embed / head).  The learning rate is a
    pure function of the 1-indexed ``run_args["step"]``.  Sharded variants (``block_params["shard"]``)
    are dispatched to ``parallel.zero``.
    """

    def layouts_for(self, ctx):
        tgt = ctx.task.block_params.get("target", "block")
        if tgt == "embed":
            return self.lay.embed_w, self.lay.embed_dw, self.lay.embed_o
        if tgt == "head":
            return self.lay.head_w, self.lay.head_dw, self.lay.head_o
        return self.lay.block_w, self.lay.block_dw, self.lay.block_o

    def run(self, ctx):
        wl, gl, ol = self.layouts_for(ctx)
        if ctx.task.block_params.get("shard"):
            from ..parallel.zero import sharded_optimizer_step
            if sharded_optimizer_step(self, ctx, wl, gl, ol, None, None, None):
                return
        w = self.views(ctx.inputs[0], wl)
        g = self.views(ctx.inputs[1], gl)
        o = self.views(ctx.inputs[2], ol) if len(ctx.inputs) > 2 else {}
        self.update_fields(ctx, wl, w, g, o)

    def update_fields(self, ctx, wl, w, g, o, rows: Mapping[str, slice] | None = None):
        hy = self.hyper
        step = int(ctx.run_args.get("step", 1))
        lr = lr_at(hy, step)
        b1, b2 = hy.get("beta1", 0.9), hy.get("beta2", 0.95)
        eps, wd = hy.get("eps", 1e-8), hy.get("weight_decay", 0.0)
        rule = hy.get("optimizer", "adamw")
        only = tuple(hy.get("train_only") or ())
        for f in wl.fields:
            if f.name not in g:
                continue            # frozen field: no gradient storage, no update
            if only and not any(fnmatch.fnmatchcase(f.name, pat) for pat in only):
                continue            # the run updates a named subset of fields only (e.g. an indexer warm-up)
            wf, gf = w[f.name], g[f.name]
            f_wd = wd if (f.kind in ("matrix", "embedding") or hy.get("wd_all")) else 0.0
            if rule == "adamw" and f"{f.name}.mlo" in o:
                self.K.adamw_split_step(wf.reshape(-1), o[f"{f.name}.mlo"].reshape(-1), gf.reshape(-1),
                                        o[f"{f.name}.s0"].reshape(-1), o[f"{f.name}.s1"].reshape(-1), lr, b1, b2, eps, f_wd, step)
            elif rule == "adamw":
                self.K.adamw_step(wf.reshape(-1), gf.reshape(-1), o[f"{f.name}.s0"].reshape(-1),
                                  o[f"{f.name}.s1"].reshape(-1), lr, b1, b2, eps, f_wd, step,
                                  master=o[f"{f.name}.master"].reshape(-1) if f"{f.name}.master" in o else None)
            elif rule in ("sgd", "sgdm"):
                self.K.sgd_step(wf.reshape(-1), gf.reshape(-1), o.get(f"{f.name}.s0").reshape(-1) if rule == "sgdm" else None,
                                lr, hy.get("momentum", 0.9), f_wd)
            elif rule == "muon":
                from .optim import muon_field_step
                muon_field_step(self.K, f, wf, gf, o, lr, hy, step)
            elif rule == "frozen":
                continue
            else:
                raise KeyError(f"unknown optimizer rule {rule!r}")


def common_executables(dims, layouts, kernels, device, hyper) -> dict[str, Any]:
    from ..parallel.zero import CommJoin, GradReduceScatter, ParamGather
    return {
        "param_gather": ParamGather(dims, layouts, kernels, device, hyper),
        "grad_rs": GradReduceScatter(dims, layouts, kernels, device, hyper),
        "grad_rs_join": CommJoin(dims, layouts, kernels, device, hyper),
        "prologue_round": RoundPrologue(dims, layouts, kernels, device, hyper),
        "embed_fwd": EmbedFwd(dims, layouts, kernels, device, hyper),
        "embed_bwd": EmbedBwd(dims, layouts, kernels, device, hyper),
        "head_loss": HeadLoss(dims, layouts, kernels, device, hyper),
        "optimizer_block": OptimizerStep(dims, layouts, kernels, device, hyper),
        "optimizer_embed": OptimizerStep(dims, layouts, kernels, device, hyper),
        "optimizer_head": OptimizerStep(dims, layouts, kernels, device, hyper),
    }
