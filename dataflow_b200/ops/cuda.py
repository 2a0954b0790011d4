"""Native lane: the hand-written sm_100a kernels (``ops/csrc``).  Registered with the
highest priority and required to exist on a Blackwell device: if the extension
is missing there, resolution raises instead of silently falling back.
"""
from __future__ import annotations

import os

import torch

from . import native, native_available
from .registry import Workspace, register

P = 10


class _LaunchCounter:
    """Counts launches of this package's own kernels (benchmarks report it)."""
    total = 0

    def reset(self):
        self.total = 0


LAUNCHES = _LaunchCounter()


def reg(op, launches=1, **kw):
    """Register a native implementation; the registered callable counts its kernel launches."""
    def deco(f):
        def counted(*a, **k):
            LAUNCHES.total += launches
            return f(*a, **k)
        counted.__name__ = f.__name__
        counted.__doc__ = f.__doc__
        register(op, "sm100", counted, priority=P, requires=_native, native=True, **kw)
        return f
    return deco


def _native(caps):
    if caps.get("sm100") and not native_available():
        native()        # raises with the build hint: no silent fallback on a B200
    return bool(caps.get("native_ops"))


def _scratch(n, device):
    return torch.empty(int(n), dtype=torch.float32, device=device)


# ------------------------------------------------------------------ norms
@reg("rmsnorm_fwd")
def rmsnorm_fwd(x, w, eps=1e-5, out=None):
    x = x.contiguous()
    rows = x.numel() // x.shape[-1]
    y = out if out is not None else torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    native().rmsnorm_fwd(x, w, y, rstd, float(eps))
    return y, rstd


@reg("rmsnorm_apply")
def rmsnorm_apply(x, w, rstd, out=None):
    y = out if out is not None else torch.empty_like(x)
    native().rmsnorm_apply(x, w, rstd, y)
    return y


@reg("rmsnorm_bwd", 2, workspace=Workspace.internal())
def rmsnorm_bwd(dy, x, w, rstd, dx_add=None, dw=None, accumulate=False, out=None):
    rows, cols = x.numel() // x.shape[-1], x.shape[-1]
    dx = out if out is not None else torch.empty_like(x)
    part = _scratch(native().norm_bwd_scratch_elems(rows, cols), x.device)
    native().rmsnorm_bwd(dy, x, w, rstd, dx, dx_add, dw, bool(accumulate), part)
    return dx


@reg("layernorm_fwd")
def layernorm_fwd(x, w, b, eps=1e-5, out=None):
    rows = x.numel() // x.shape[-1]
    y = out if out is not None else torch.empty_like(x)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    native().layernorm_fwd(x, w, b, y, mean, rstd, float(eps))
    return y, mean, rstd


@reg("layernorm_apply")
def layernorm_apply(x, w, b, mean, rstd, out=None):
    y = out if out is not None else torch.empty_like(x)
    native().layernorm_apply(x, w, b, mean, rstd, y)
    return y


@reg("layernorm_bwd", 2, workspace=Workspace.internal())
def layernorm_bwd(dy, x, w, mean, rstd, dx_add=None, dw=None, db=None, accumulate=False, out=None):
    rows, cols = x.numel() // x.shape[-1], x.shape[-1]
    dx = out if out is not None else torch.empty_like(x)
    part = _scratch(native().norm_bwd_scratch_elems(rows, cols), x.device)
    native().layernorm_bwd(dy, x, w, mean, rstd, dx, dx_add, dw, db, bool(accumulate), part)
    return dx


# ------------------------------------------------------------------ rope (x: (tokens, heads, head_dim) view, inner stride 1)
def _rope(x, positions, theta, rot_dim, col_base, backward):
    assert x.dim() == 3 and x.stride(2) == 1
    native().rope_inplace(x, positions, x.shape[1], rot_dim or x.shape[2], x.stride(0), x.stride(1), col_base,
                          float(theta), backward)
    return x


@reg("rope_fwd")
def rope_fwd(x, positions, theta, rot_dim=None, col_base=0):
    return _rope(x, positions, theta, rot_dim, col_base, False)


@reg("rope_bwd")
def rope_bwd(x, positions, theta, rot_dim=None, col_base=0):
    return _rope(x, positions, theta, rot_dim, col_base, True)


# ------------------------------------------------------------------ activations
def _rows_ld(t):
    assert t.stride(-1) == 1
    F = t.shape[-1]
    rows = t.numel() // F
    ld = t.stride(-2) if t.dim() >= 2 else F
    return rows, F, ld


@reg("swiglu_fwd_out")
def swiglu_fwd_out(x1, x3, out=None):
    rows, F, ld1 = _rows_ld(x1)
    _, _, ld3 = _rows_ld(x3)
    if out is None:
        out = torch.empty(*x1.shape, dtype=x1.dtype, device=x1.device)
    native().swiglu_fwd(x1, x3, out, rows, F, ld1, ld3)
    return out


@reg("swiglu_bwd")
def swiglu_bwd(ds, x1, x3, dx1=None, dx3=None, s_out=None):
    rows, F, ld1 = _rows_ld(x1)
    _, _, ld3 = _rows_ld(x3)
    if dx1 is None:
        dx1 = torch.empty(*x1.shape, dtype=x1.dtype, device=x1.device)
    if dx3 is None:
        dx3 = torch.empty(*x3.shape, dtype=x3.dtype, device=x3.device)
    native().swiglu_bwd(ds, x1, x3, dx1, dx3, rows, F, ld1, ld3, _rows_ld(dx1)[2], _rows_ld(dx3)[2], s_out)
    return dx1, dx3


@reg("swiglu_packed_fwd")
def swiglu_packed_fwd(h13, out=None):
    F = h13.shape[-1] // 2
    return swiglu_fwd_out(h13[..., :F], h13[..., F:], out)


@reg("swiglu_packed_bwd")
def swiglu_packed_bwd(ds, h13, dh13=None, with_s=False):
    """dh13 from ds; ``with_s``: also the forward product s = silu(x1) * x3 (the same bytes ``swiglu_packed_fwd`` gives),
    written by the same launch."""
    F = h13.shape[-1] // 2
    if dh13 is None:
        dh13 = torch.empty_like(h13)
    s = torch.empty(*h13.shape[:-1], F, dtype=h13.dtype, device=h13.device) if with_s else None
    swiglu_bwd(ds, h13[..., :F], h13[..., F:], dh13[..., :F], dh13[..., F:], s)
    return (dh13, s) if with_s else dh13


@reg("gelu_fwd_out")
def gelu_fwd_out(x, out=None):
    out = out if out is not None else torch.empty_like(x)
    native().gelu_fwd(x, out)
    return out


@reg("gelu_bwd")
def gelu_bwd(dy, x, out=None):
    out = out if out is not None else torch.empty_like(x)
    native().gelu_bwd(dy, x, out)
    return out


@reg("add")
def add(a, b, out=None):
    out = out if out is not None else torch.empty_like(a)
    native().add_bf16(a, b, out)
    return out


# ------------------------------------------------------------------ loss / embedding
@reg("ce_loss_fwd_bwd", 2, workspace=Workspace.internal())
def ce_loss_fwd_bwd(logits, targets, total_rows, loss_out=None, accumulate=False):
    nll = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
    if loss_out is None:
        loss_out = torch.zeros(1, dtype=torch.float32, device=logits.device)
        accumulate = False
    native().ce_loss_fwd_bwd(logits, targets, nll, loss_out, bool(accumulate), 1.0 / float(total_rows))
    return loss_out


@reg("embed_fwd")
def embed_fwd(tok, table, out=None, positions=None, pos_table=None):
    if out is None:
        out = torch.empty(tok.numel(), table.shape[1], dtype=table.dtype, device=table.device)
    native().embed_fwd(tok, table, out, positions, pos_table)
    return out


@reg("embed_bwd_accum", workspace=Workspace.internal())
def embed_bwd_accum(tok, dy, dtable, accumulate=False):
    if not accumulate:
        dtable.zero_()
    sorted_tok, order = torch.sort(tok, stable=True)
    native().embed_bwd_sorted(sorted_tok.int(), order.int(), dy, dtable, True)
    return dtable


# ------------------------------------------------------------------ optimizers
@reg("adamw_step")
def adamw_step(w, g, m, v, lr, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.0, step=1, master=None, gscale=1.0):
    if master is not None:
        native().adamw_master(master, w, g, m, v, lr, beta1, beta2, eps, wd, int(step), gscale)
    elif w.dtype == torch.float32:
        native().adamw_f32(w, g, m, v, lr, beta1, beta2, eps, wd, int(step), gscale)
    else:
        native().adamw_bf16(w, g, m, v, lr, beta1, beta2, eps, wd, int(step), gscale)
    return w


@reg("adamw_split_step")
def adamw_split_step(w, lo, g, m, v, lr, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.0, step=1, gscale=1.0):
    native().adamw_split(w, lo, g, m, v, lr, beta1, beta2, eps, wd, int(step), gscale)
    return w


@reg("sgd_step")
def sgd_step(w, g, m=None, lr=1e-2, momentum=0.0, wd=0.0):
    native().sgd_bf16(w, g, m, lr, momentum, wd)
    return w


# ------------------------------------------------------------------ linear triple on the tcgen05 GEMM (W stored (in, out))
@reg("linear_fwd_bf16")
def linear_fwd(x, w, out=None, add=None, bias=None):
    if out is None:
        out = torch.empty(x.shape[0], w.shape[1], dtype=x.dtype, device=x.device)
    native().gemm_bf16(x, False, w, True, out, add, bias)          # A (M,K) K-major; B stored (K,N): N-major
    return out


@reg("linear_dgrad_bf16")
def linear_dgrad(dy, w, out=None, add=None):
    if out is None:
        out = torch.empty(dy.shape[0], w.shape[0], dtype=dy.dtype, device=dy.device)
    native().gemm_bf16(dy, False, w, False, out, add, None)        # B = W as (N_out=in, K_red=out): K-major
    return out


@reg("linear_wgrad_bf16")
def linear_wgrad(x, dy, dw, accumulate=False):
    native().gemm_bf16(x, True, dy, True, dw, dw if accumulate else None, None)   # both operands token-major
    return dw


@reg("bias_grad", 2, workspace=Workspace.internal())
def bias_grad(dy, db, accumulate=False):
    dy2 = dy.reshape(-1, dy.shape[-1])
    part = _scratch(native().colsum_parts(dy2.shape[0]) * dy2.shape[1], dy.device)
    native().colsum_bf16(dy2, part, db, bool(accumulate))
    return db


# ------------------------------------------------------------------ mixture of experts
@reg("moe_topk_softmax")
def moe_topk_softmax(logits, top_k: int, mode: str = "topk_then_softmax"):
    t = logits.shape[0]
    w = torch.empty(t, top_k, dtype=torch.float32, device=logits.device)
    ids = torch.empty(t, top_k, dtype=torch.int32, device=logits.device)
    native().moe_topk_softmax(logits.contiguous(), w, ids, mode)
    return w, ids


@reg("moe_router_bwd")
def moe_router_bwd(dprob, route_w, route_ids, logits, mode: str = "topk_then_softmax"):
    out = torch.empty(logits.shape, dtype=torch.float32, device=logits.device)
    native().moe_router_bwd(dprob.float().contiguous(), route_w.float().contiguous(), route_ids.contiguous(), logits.contiguous(),
                            out, mode)
    return out


@reg("moe_dispatch")
def moe_dispatch(x, row_src, out=None):
    xp = out if out is not None else torch.empty(row_src.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
    native().moe_dispatch(x, row_src, xp)
    return xp


@reg("moe_combine")
def moe_combine(base, yp, route_w, row_of, out=None):
    y = out if out is not None else torch.empty(row_of.shape[0], yp.shape[1], dtype=yp.dtype, device=yp.device)
    native().moe_combine(base, yp, route_w.float().contiguous(), row_of, y)
    return y


@reg("moe_dispatch_bwd")
def moe_dispatch_bwd(dxp, row_of, out=None, accumulate: bool = False):
    if out is None:
        out = torch.empty(row_of.shape[0], dxp.shape[1], dtype=dxp.dtype, device=dxp.device)
        accumulate = False
    native().moe_dispatch_bwd(dxp, row_of, out, bool(accumulate))
    return out


@reg("moe_scale_rows")
def moe_scale_rows(xp, route_w, row_of):
    native().moe_scale_rows(xp, route_w.float().contiguous(), row_of)
    return xp


@reg("moe_rowdot")
def moe_rowdot(a, b, row_of):
    out = torch.empty(row_of.shape, dtype=torch.float32, device=a.device)
    native().moe_rowdot(a, b, row_of, out)
    return out


@reg("moe_sort", launches=3)
def moe_sort(route_ids, n_experts: int, tile_rows: int = 256):
    """The padded expert-major layout by a stable counting sort on the device (three small kernels, no library sort)."""
    t, k = route_ids.shape
    n = t * k
    if n_experts > 1024 or n == 0:
        from . import eager
        return eager.moe_sort(route_ids, n_experts, tile_rows)
    dev = route_ids.device
    mp = (n + tile_rows - 1) // tile_rows * tile_rows + n_experts * tile_rows
    i32 = dict(dtype=torch.int32, device=dev)
    row_of, row_src = torch.empty(t, k, **i32), torch.empty(mp, **i32)
    offsets_pad, tile_expert, counts = torch.empty(n_experts + 1, **i32), torch.empty(mp // tile_rows, **i32), torch.empty(n_experts, **i32)
    scratch = torch.empty(((n + 1023) // 1024) * n_experts, **i32)
    native().moe_sort(route_ids.to(torch.int32).contiguous(), int(n_experts), int(tile_rows), row_of, row_src, offsets_pad, tile_expert, counts, scratch)
    return row_of, row_src, offsets_pad, tile_expert, counts


@reg("moe_grouped_mm")
def moe_grouped_mm(xp, w, tile_expert, out=None, transpose_w: bool = False):
    """``tile_expert``: the per-row-tile expert table of ``moe_sort`` (device int32)."""
    n = w.shape[1] if transpose_w else w.shape[2]
    y = out if out is not None else torch.empty(xp.shape[0], n, dtype=xp.dtype, device=xp.device)
    native().moe_grouped_mm(xp, w, y, tile_expert, not transpose_w)
    return y


@reg("moe_grouped_wgrad", launches=2)
def moe_grouped_wgrad(xp, dyp, offsets_pad, dw, accumulate: bool = False):
    native().moe_grouped_wgrad(xp, dyp, dw, offsets_pad, bool(accumulate))
    return dw


# ------------------------------------------------------------------ sparse-attention indexer (dsa.cu)
@reg("dsa_index_scores")
def dsa_index_scores(q, k, wgt, seg_start, q0: int, q1: int, key_lo: int):
    D = q.shape[-1]
    if q.dtype != torch.bfloat16 or D not in (64, 128):
        from . import eager
        return eager.dsa_index_scores(q, k, wgt, seg_start, q0, q1, key_lo)
    out = torch.empty(q1 - q0, q1 - key_lo, dtype=torch.float32, device=q.device)
    native().dsa_index_scores(q.contiguous(), k.contiguous(), wgt.float().contiguous(), seg_start.to(torch.int32).contiguous(), out,
                              int(q0), int(q1), int(key_lo))
    return out


@reg("dsa_topk_rows")
def dsa_topk_rows(scores, k: int, col_base: int = 0):
    rows, cols = scores.shape
    sel = torch.empty(rows, k, dtype=torch.int32, device=scores.device)
    native().dsa_topk_rows(scores.float().contiguous(), rows, cols, int(col_base), int(k), sel)
    return sel


# ------------------------------------------------------------------ sequence-mixing helpers (seqmix.cu)
@reg("l2norm_fwd")
def l2norm_fwd(x, eps: float = 1e-6):
    xc = x.contiguous()
    y = torch.empty_like(xc)
    rstd = torch.empty(xc.numel() // xc.shape[-1], dtype=torch.float32, device=x.device)
    native().l2norm_fwd(xc, y, rstd, float(eps))
    return y, rstd


@reg("l2norm_bwd")
def l2norm_bwd(dy, x, rstd):
    dx = torch.empty_like(x, memory_format=torch.contiguous_format)
    native().l2norm_bwd(dy.contiguous(), x.contiguous(), rstd, dx)
    return dx


@reg("gated_rmsnorm_fwd")
def gated_rmsnorm_fwd(x, g, w, eps: float = 1e-6):
    xc = x.contiguous()
    y = torch.empty_like(xc)
    rstd = torch.empty(xc.numel() // xc.shape[-1], dtype=torch.float32, device=x.device)
    native().gated_rmsnorm_fwd(xc, g.contiguous(), w.contiguous(), y, rstd, float(eps))
    return y, rstd


@reg("gated_rmsnorm_bwd", 2)
def gated_rmsnorm_bwd(dy, x, g, w, rstd):
    xc = x.contiguous()
    dx, dg = torch.empty_like(xc), torch.empty_like(xc)
    rows = xc.numel() // xc.shape[-1]
    blocks = max(min((rows + 7) // 8, 296), 1)
    part = torch.empty(blocks, xc.shape[-1], dtype=torch.float32, device=x.device)
    native().gated_rmsnorm_bwd(dy.contiguous(), xc, g.contiguous(), w.contiguous(), rstd, dx, dg, part)
    return dx, dg, part.sum(0)


@reg("conv_silu_fwd")
def conv_silu_fwd(x, w, seg_start):
    y = torch.empty_like(x, memory_format=torch.contiguous_format)
    native().conv_silu_fwd(x.contiguous(), w.contiguous(), seg_start.to(torch.int32), y)
    return y


@reg("conv_silu_bwd", 2)
def conv_silu_bwd(dy, x, w, seg_start):
    n, c = x.shape
    rows_per_block = 64
    blocks = max((n + rows_per_block - 1) // rows_per_block, 1)
    dx = torch.empty_like(x, memory_format=torch.contiguous_format)
    part = torch.empty(blocks, c, w.shape[1], dtype=torch.float32, device=x.device)
    native().conv_silu_bwd(dy.contiguous(), x.contiguous(), w.contiguous(), seg_start.to(torch.int32), dx, part, rows_per_block)
    return dx, part.sum(0)


@reg("moe_topk_sigmoid_noaux")
def moe_topk_sigmoid_noaux(logits, bias, top_k: int, n_group: int = 1, topk_group: int = 1, routed_scaling: float = 1.0,
                           norm_topk: bool = True):
    if not norm_topk:
        raise NotImplementedError("the native router normalises the selected weights")
    t = logits.shape[0]
    w = torch.empty(t, top_k, dtype=torch.float32, device=logits.device)
    ids = torch.empty(t, top_k, dtype=torch.int32, device=logits.device)
    native().router_sigmoid_noaux(logits.to(torch.bfloat16).contiguous(), bias.float().contiguous(), w, ids, int(n_group), int(topk_group),
                                  float(routed_scaling))
    return w, ids


# ------------------------------------------------------------------ fp8 lane (fp8.cu, gemm_tcgen05_2sm.cu FP8)
@reg("quant_fp8_rowwise")
def quant_fp8_rowwise(x):
    q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    scale = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
    native().quant_fp8_rowwise(x, q, scale)
    return q, scale


@reg("linear_fp8")
def linear_fp8(xq, x_scale, wq, w_scale, out=None, add=None, bias=None, out_dtype=torch.bfloat16):
    if out is None:
        out = torch.empty(xq.shape[0], wq.shape[0], dtype=out_dtype, device=xq.device)
    native().gemm_fp8(xq, wq, out, x_scale, w_scale, add, bias)
    return out


@reg("linear_fwd_fp8", launches=3)
def linear_fwd_fp8(x, w, out=None, add=None, bias=None):
    """Forward linear on the fp8 tensor-core path: quantise x per row and w (stored (in, out)) per output column, run the
    ``kind::f8f6f4`` GEMM, dequantise in its epilogue.  The weight is transposed to (out, in) on the way (one copy)."""
    xq, sx = quant_fp8_rowwise(x)
    wq, sw = quant_fp8_rowwise(w.t().contiguous())
    return linear_fp8(xq, sx, wq, sw, out=out, add=add, bias=bias, out_dtype=out.dtype if out is not None else x.dtype)


# ------------------------------------------------------------------ attention forward on tcgen05 (attention.cu)
def flash_fwd_tcgen05(q, k, v, cu_seqlens, max_seqlen, scale=None, out=None):
    """Causal varlen attention on the hand-written kernel, head_dim 128; q (t, hq, 128), k / v (t, hkv, 128) — views into a
    packed qkv are taken as they are.  Returns (out (t, hq, 128), lse (hq, t))."""
    LAUNCHES.total += 1
    scale = scale if scale is not None else q.shape[-1] ** -0.5
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    lse = torch.empty(q.shape[1], q.shape[0], dtype=torch.float32, device=q.device)
    native().flash_fwd(q, k, v, out, lse, cu_seqlens.to(torch.int32), int(max_seqlen), float(scale))
    return out, lse


def _own_attention(q) -> bool:
    """Shapes the hand-written attention kernels take: bf16, head_dim 128, heads contiguous inside a token row."""
    return q.shape[-1] == 128 and q.dtype == torch.bfloat16 and q.stride(2) == 1 and q.stride(1) == 128


def _flash_fwd(q, k, v, cu_seqlens, max_seqlen, scale=None, out=None):
    """Attention forward of the default lane: the tcgen05 kernel of this repository for head_dim 128 (uniform and ragged
    rounds alike).  Other head sizes, and every round when ``DFB_ATTN_FWD=library`` is set, go to the vendor kernels of the
    baseline lane."""
    from . import library
    if _own_attention(q) and os.environ.get("DFB_ATTN_FWD") != "library":
        return flash_fwd_tcgen05(q, k, v, cu_seqlens, max_seqlen, scale, out)
    return library.flash_fwd(q, k, v, cu_seqlens, max_seqlen, scale, out)


def flash_bwd_tcgen05(dout, q, k, v, out, lse, cu_seqlens, max_seqlen, scale=None, dq=None, dk=None, dv=None):
    """Causal varlen attention backward on the hand-written kernels (attention_bwd.cu): deterministic, GQA summed inside the
    dK / dV kernel.  Gradient buffers may be views into a packed (tokens, (hq + 2 hkv) * 128) buffer."""
    LAUNCHES.total += 3
    scale = scale if scale is not None else q.shape[-1] ** -0.5
    dq = torch.empty(q.shape, dtype=q.dtype, device=q.device) if dq is None else dq
    dk = torch.empty(k.shape, dtype=k.dtype, device=k.device) if dk is None else dk
    dv = torch.empty(v.shape, dtype=v.dtype, device=v.device) if dv is None else dv
    scratch = torch.empty(2 * q.shape[1] * q.shape[0], dtype=torch.float32, device=q.device)
    native().flash_bwd(dout, q, k, v, out, lse, dq, dk, dv, scratch, cu_seqlens.to(torch.int32), int(max_seqlen), float(scale))
    return dq, dk, dv


def _flash_bwd(dout, q, k, v, out, lse, cu_seqlens, max_seqlen, scale=None, dq=None, dk=None, dv=None):
    from . import library
    ok = _own_attention(q) and all(t is None or (t.stride(-1) == 1 and t.stride(1) == 128) for t in (dq, dk, dv)) and \
        dout.stride(2) == 1 and dout.stride(1) == 128 and out.stride(2) == 1 and out.stride(1) == 128
    if ok and os.environ.get("DFB_ATTN_BWD") != "library":
        return flash_bwd_tcgen05(dout, q, k, v, out, lse, cu_seqlens, max_seqlen, scale, dq, dk, dv)
    return library.flash_bwd(dout, q, k, v, out, lse, cu_seqlens, max_seqlen, scale, dq, dk, dv)


register("flash_fwd", "sm100", _flash_fwd, priority=P, requires=_native, native=True)
register("flash_bwd", "sm100", _flash_bwd, priority=P, requires=_native, native=True, workspace=Workspace.internal())
