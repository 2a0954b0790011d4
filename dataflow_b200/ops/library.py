"""Library lane ("baseline"): vendor-library implementations kept as the A/B
baseline and as a stop-gap where no hand-written kernel exists yet — cuBLAS
GEMMs through ``torch.matmul`` and the aten flash-attention kernels.  Role
parity: reference ``src/dataflow_training/blocks/linear.py:58-90`` and
``kernels/flash.py:59-172`` (these *are* the reference's hot path).
"""
from __future__ import annotations

import torch

from .registry import register


def _cuda(caps):
    return bool(caps.get("cuda"))


@register("linear_fwd_bf16", "baseline", priority=5, requires=_cuda)
def linear_fwd(x, w, out=None, add=None, bias=None):
    if out is None:
        out = torch.empty(x.shape[0], w.shape[1], dtype=x.dtype, device=x.device)
    if add is not None:
        if bias is not None:
            torch.addmm(bias, x, w, out=out)
            out.add_(add)
        else:
            torch.addmm(add, x, w, out=out)
    elif bias is not None:
        torch.addmm(bias, x, w, out=out)
    else:
        torch.matmul(x, w, out=out)
    return out


@register("linear_dgrad_bf16", "baseline", priority=5, requires=_cuda)
def linear_dgrad(dy, w, out=None, add=None):
    if out is None:
        out = torch.empty(dy.shape[0], w.shape[0], dtype=dy.dtype, device=dy.device)
    if add is not None:
        torch.addmm(add, dy, w.t(), out=out)
    else:
        torch.matmul(dy, w.t(), out=out)
    return out


@register("linear_wgrad_bf16", "baseline", priority=5, requires=_cuda)
def linear_wgrad(x, dy, dw, accumulate=False):
    if dw.dtype != x.dtype:
        g = torch.matmul(x.t(), dy)
        if accumulate:
            dw.add_(g)
        else:
            dw.copy_(g)
        return dw
    if accumulate:
        dw.addmm_(x.t(), dy)
    else:
        torch.matmul(x.t(), dy, out=dw)
    return dw


@register("flash_fwd", "baseline", priority=5, requires=_cuda)
def flash_fwd(q, k, v, cu_seqlens, max_seqlen, scale=None, out=None):
    """aten varlen flash attention; q (t, hq, d).  Returns (out, lse (hq, t))."""
    scale = scale if scale is not None else q.shape[-1] ** -0.5
    res = torch.ops.aten._flash_attention_forward(q, k, v, cu_seqlens, cu_seqlens, int(max_seqlen), int(max_seqlen),
                                                  0.0, True, False, scale=scale)
    o, lse = res[0], res[1]
    if out is not None:
        out.copy_(o)
        o = out
    return o, lse


@register("flash_bwd", "baseline", priority=5, requires=_cuda)
def flash_bwd(dout, q, k, v, out, lse, cu_seqlens, max_seqlen, scale=None, dq=None, dk=None, dv=None):
    scale = scale if scale is not None else q.shape[-1] ** -0.5
    z = torch.zeros(2, dtype=torch.uint64, device=q.device) if hasattr(torch, "uint64") else torch.zeros(2, dtype=torch.int64, device=q.device)
    gq, gk, gv = torch.ops.aten._flash_attention_backward(dout, q, k, v, out, lse, cu_seqlens, cu_seqlens,
                                                          int(max_seqlen), int(max_seqlen), 0.0, True, z[0], z[1],
                                                          scale=scale)
    res = []
    for buf, val in ((dq, gq), (dk, gk), (dv, gv)):
        if buf is not None:
            buf.copy_(val)
            val = buf
        res.append(val)
    return tuple(res)
