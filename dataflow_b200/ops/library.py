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


# Attention runs on vendor kernels in this lane: for rounds whose sequences all have the same length (the packed
# benchmark shape) cuDNN's fused attention, which uses the tensor cores of the device generation it runs on; otherwise
# (ragged rounds) aten's varlen flash attention.  ``DFB_ATTN=flash`` pins the latter.  Both produce the same
# saved statistics: lse (heads, tokens), natural log, scale applied.
import os as _os

_CUDNN = {"ok": _os.environ.get("DFB_ATTN", "cudnn") != "flash"}


def _uniform(q, cu_seqlens, max_seqlen) -> int:
    """Number of equal-length sequences in the round, or 0 when it is ragged (host-known shapes only: no sync)."""
    nseg = cu_seqlens.numel() - 1
    return nseg if _CUDNN["ok"] and nseg * int(max_seqlen) == q.shape[0] and q.shape[-1] % 8 == 0 and max_seqlen % 64 == 0 else 0


def _bhsd(t, b, s):
    """(tokens, heads, d) view -> (batch, heads, seq, d) view over the same memory."""
    return t.unflatten(0, (b, s)).transpose(1, 2)


@register("flash_fwd", "baseline", priority=5, requires=_cuda)
def flash_fwd(q, k, v, cu_seqlens, max_seqlen, scale=None, out=None):
    """Causal varlen attention; q (t, hq, d), k / v (t, hkv, d).  Returns (out (t, hq, d), lse (hq, t))."""
    scale = scale if scale is not None else q.shape[-1] ** -0.5
    b = _uniform(q, cu_seqlens, max_seqlen)
    if b:
        s_ = int(max_seqlen)
        try:
            r = torch.ops.aten._scaled_dot_product_cudnn_attention(_bhsd(q, b, s_), _bhsd(k, b, s_), _bhsd(v, b, s_), None, True, 0.0,
                                                                   True, False, scale=scale)
        except RuntimeError:
            _CUDNN["ok"] = False                      # this build of the library cannot run the shape: use flash from now on
        else:
            o = r[0].transpose(1, 2).reshape(q.shape)                                   # stored (b, s, h, d): a view
            lse = r[1].view(b, q.shape[1], s_).permute(1, 0, 2).reshape(q.shape[1], q.shape[0])
            if out is not None:
                out.copy_(o)
                o = out
            return o, lse
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
    b = _uniform(q, cu_seqlens, max_seqlen)
    grads = None
    if b:
        s_ = int(max_seqlen)
        lse4 = lse.view(q.shape[1], b, s_).permute(1, 0, 2).unsqueeze(-1).contiguous()
        try:
            g4 = torch.ops.aten._scaled_dot_product_cudnn_attention_backward(
                _bhsd(dout, b, s_), _bhsd(q, b, s_), _bhsd(k, b, s_), _bhsd(v, b, s_), _bhsd(out, b, s_), lse4, z[0], z[1], None,
                None, None, s_, s_, 0.0, True, scale=scale)
            grads = tuple(x.transpose(1, 2).reshape(y.shape) for x, y in zip(g4, (q, k, v)))
        except RuntimeError:
            _CUDNN["ok"] = False
    if grads is None:
        grads = torch.ops.aten._flash_attention_backward(dout, q, k, v, out, lse, cu_seqlens, cu_seqlens,
                                                         int(max_seqlen), int(max_seqlen), 0.0, True, z[0], z[1], scale=scale)
    res = []
    for buf, val in zip((dq, dk, dv), grads):
        if buf is not None:
            buf.copy_(val)
            val = buf
        res.append(val)
    return tuple(res)
