"""Pure-PyTorch reference lane ("eager"): the oracle of every numerics test and the
math path on machines without a GPU.  Runs on CPU or CUDA tensors of any float
dtype; all reductions and elementwise math are done in fp32 and rounded once to
the storage dtype.  Numerics follow the reference's eager ops
(``src/dataflow_training/blocks/ops.py:30-500``).
"""
from __future__ import annotations

import math

import torch

from .registry import register

RMS_EPS = 1e-5


def _st(x, ref):
    return x.to(ref.dtype)


# ------------------------------------------------------------------ norms
@register("rmsnorm_fwd", "eager")
def rmsnorm_fwd(x, w, eps=RMS_EPS, out=None):
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
    y = xf * rstd.unsqueeze(-1)
    if w is not None:
        y = y * w.float()
    y = _st(y, x)
    if out is not None:
        out.copy_(y)
        y = out
    return y, rstd.reshape(-1)


@register("rmsnorm_apply", "eager")
def rmsnorm_apply(x, w, rstd, out=None):
    y = _st(x.float() * rstd.reshape(*x.shape[:-1], 1) * w.float(), x)
    if out is not None:
        out.copy_(y)
        return out
    return y


@register("rmsnorm_bwd", "eager")
def rmsnorm_bwd(dy, x, w, rstd, dx_add=None, dw=None, accumulate=False, out=None):
    xf, g = x.float(), dy.float() * w.float()
    r = rstd.reshape(*x.shape[:-1], 1)
    xh = xf * r
    dx = (g - xh * (g * xh).mean(-1, keepdim=True)) * r
    if dx_add is not None:
        dx = dx + dx_add.float()
    if dw is not None:
        gw = (dy.float() * xh).reshape(-1, x.shape[-1]).sum(0)
        dw.copy_(_st(gw + (dw.float() if accumulate else 0), dw))
    dx = _st(dx, x)
    if out is not None:
        out.copy_(dx)
        return out
    return dx


@register("layernorm_fwd", "eager")
def layernorm_fwd(x, w, b, eps=RMS_EPS, out=None):
    xf = x.float()
    mean = xf.mean(-1)
    var = (xf - mean.unsqueeze(-1)).pow(2).mean(-1)
    rstd = torch.rsqrt(var + eps)
    y = (xf - mean.unsqueeze(-1)) * rstd.unsqueeze(-1) * w.float()
    if b is not None:
        y = y + b.float()
    y = _st(y, x)
    if out is not None:
        out.copy_(y)
        y = out
    return y, mean.reshape(-1), rstd.reshape(-1)


@register("layernorm_apply", "eager")
def layernorm_apply(x, w, b, mean, rstd, out=None):
    sh = (*x.shape[:-1], 1)
    y = (x.float() - mean.reshape(sh)) * rstd.reshape(sh) * w.float()
    if b is not None:
        y = y + b.float()
    y = _st(y, x)
    if out is not None:
        out.copy_(y)
        return out
    return y


@register("layernorm_bwd", "eager")
def layernorm_bwd(dy, x, w, mean, rstd, dx_add=None, dw=None, db=None, accumulate=False, out=None):
    sh = (*x.shape[:-1], 1)
    xh = (x.float() - mean.reshape(sh)) * rstd.reshape(sh)
    g = dy.float() * w.float()
    dx = (g - g.mean(-1, keepdim=True) - xh * (g * xh).mean(-1, keepdim=True)) * rstd.reshape(sh)
    if dx_add is not None:
        dx = dx + dx_add.float()
    if dw is not None:
        gw = (dy.float() * xh).reshape(-1, x.shape[-1]).sum(0)
        dw.copy_(_st(gw + (dw.float() if accumulate else 0), dw))
    if db is not None:
        gb = dy.float().reshape(-1, x.shape[-1]).sum(0)
        db.copy_(_st(gb + (db.float() if accumulate else 0), db))
    dx = _st(dx, x)
    if out is not None:
        out.copy_(dx)
        return out
    return dx


# ------------------------------------------------------------------ rope
def _rope(x, positions, theta, rot_dim, col_base, sign):
    """x: (tokens, heads, head_dim) view (any strides); rotate-half on [col_base, col_base+rot_dim)."""
    half = rot_dim // 2
    inv = torch.exp2(-math.log2(theta) * (2.0 * torch.arange(half, device=x.device, dtype=torch.float32) / rot_dim))
    ang = positions.float().unsqueeze(-1) * inv
    cs, sn = torch.cos(ang).unsqueeze(1), (torch.sin(ang) * sign).unsqueeze(1)
    a = x[..., col_base:col_base + half].float()
    b = x[..., col_base + half:col_base + rot_dim].float()
    lo, hi = _st(a * cs - b * sn, x), _st(b * cs + a * sn, x)     # both halves before either is overwritten
    x[..., col_base:col_base + half] = lo
    x[..., col_base + half:col_base + rot_dim] = hi
    return x


@register("rope_fwd", "eager")
def rope_fwd(x, positions, theta, rot_dim=None, col_base=0):
    return _rope(x, positions, theta, rot_dim or x.shape[-1], col_base, 1.0)


@register("rope_bwd", "eager")
def rope_bwd(x, positions, theta, rot_dim=None, col_base=0):
    return _rope(x, positions, theta, rot_dim or x.shape[-1], col_base, -1.0)


# ------------------------------------------------------------------ attention
def attention_reference(q, k, v, cu_seqlens, scale=None, causal=True):
    """Varlen causal GQA attention in fp32.  q (t, hq, d), k (t, hkv, d), v (t, hkv, dv).
    Returns out (t, hq, dv) in q's dtype and lse (hq, t) fp32."""
    t, hq, d = q.shape
    hkv, dv = k.shape[1], v.shape[-1]
    rep = hq // hkv
    scale = scale if scale is not None else d ** -0.5
    out = torch.empty(t, hq, dv, dtype=torch.float32, device=q.device)
    lse = torch.empty(hq, t, dtype=torch.float32, device=q.device)
    cu = [int(c) for c in cu_seqlens.tolist()] if torch.is_tensor(cu_seqlens) else list(cu_seqlens)
    for s, e in zip(cu[:-1], cu[1:]):
        if e <= s:
            continue
        qs = q[s:e].float().transpose(0, 1)                                 # (hq, L, d)
        ks = k[s:e].float().transpose(0, 1).repeat_interleave(rep, 0)
        vs = v[s:e].float().transpose(0, 1).repeat_interleave(rep, 0)
        sc = torch.matmul(qs, ks.transpose(1, 2)) * scale
        if causal:
            L = e - s
            mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
            sc = sc.masked_fill(~mask, float("-inf"))
        l = torch.logsumexp(sc, -1)
        p = torch.exp(sc - l.unsqueeze(-1))
        out[s:e] = torch.matmul(p, vs).transpose(0, 1)
        lse[:, s:e] = l
    return out.to(q.dtype), lse


@register("flash_fwd", "eager")
def flash_fwd(q, k, v, cu_seqlens, max_seqlen, scale=None, out=None):
    o, lse = attention_reference(q, k, v, cu_seqlens, scale)
    if out is not None:
        out.copy_(o)
        o = out
    return o, lse


@register("flash_bwd", "eager")
def flash_bwd(dout, q, k, v, out, lse, cu_seqlens, max_seqlen, scale=None, dq=None, dk=None, dv=None):
    t, hq, d = q.shape
    hkv = k.shape[1]
    rep = hq // hkv
    scale = scale if scale is not None else d ** -0.5
    dq_ = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    dk_ = torch.zeros(k.shape, dtype=torch.float32, device=q.device)
    dv_ = torch.zeros(v.shape, dtype=torch.float32, device=q.device)
    cu = [int(c) for c in cu_seqlens.tolist()] if torch.is_tensor(cu_seqlens) else list(cu_seqlens)
    for s, e in zip(cu[:-1], cu[1:]):
        if e <= s:
            continue
        L = e - s
        qs = q[s:e].float().transpose(0, 1)
        ks = k[s:e].float().transpose(0, 1).repeat_interleave(rep, 0)
        vs = v[s:e].float().transpose(0, 1).repeat_interleave(rep, 0)
        do = dout[s:e].float().transpose(0, 1)
        o = out[s:e].float().transpose(0, 1)
        sc = torch.matmul(qs, ks.transpose(1, 2)) * scale
        mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
        sc = sc.masked_fill(~mask, float("-inf"))
        p = torch.exp(sc - lse[:, s:e].unsqueeze(-1))
        dvs = torch.matmul(p.transpose(1, 2), do)
        dp = torch.matmul(do, vs.transpose(1, 2))
        delta = (do * o).sum(-1, keepdim=True)
        ds = p * (dp - delta) * scale
        dq_[s:e] = torch.matmul(ds, ks).transpose(0, 1)
        dks = torch.matmul(ds.transpose(1, 2), qs)
        dk_[s:e] = dks.reshape(hkv, rep, L, d).sum(1).transpose(0, 1)
        dv_[s:e] = dvs.reshape(hkv, rep, L, v.shape[-1]).sum(1).transpose(0, 1)
    res = []
    for buf, val, ref in ((dq, dq_, q), (dk, dk_, k), (dv, dv_, v)):
        val = val.to(ref.dtype)
        if buf is not None:
            buf.copy_(val)
            val = buf
        res.append(val)
    return tuple(res)


# ------------------------------------------------------------------ activations
def _silu_st(x1):
    return (x1.float() * torch.sigmoid(x1.float())).to(x1.dtype).float()


@register("swiglu_fwd_out", "eager")
def swiglu_fwd_out(x1, x3, out=None):
    y = _st(_silu_st(x1) * x3.float(), x1)
    if out is not None:
        out.copy_(y)
        return out
    return y


@register("swiglu_bwd", "eager")
def swiglu_bwd(ds, x1, x3, dx1=None, dx3=None):
    f1, f3, g = x1.float(), x3.float(), ds.float()
    sg = torch.sigmoid(f1)
    sl = f1 * sg
    d1 = _st(g * f3 * (sg + sl * (1 - sg)), x1)
    d3 = _st(g * sl, x1)
    if dx1 is not None:
        dx1.copy_(d1)
        d1 = dx1
    if dx3 is not None:
        dx3.copy_(d3)
        d3 = dx3
    return d1, d3


@register("swiglu_packed_fwd", "eager")
def swiglu_packed_fwd(h13, out=None):
    F = h13.shape[-1] // 2
    return swiglu_fwd_out(h13[..., :F], h13[..., F:], out)


@register("swiglu_packed_bwd", "eager")
def swiglu_packed_bwd(ds, h13, dh13=None, with_s=False):
    F = h13.shape[-1] // 2
    if dh13 is None:
        dh13 = torch.empty_like(h13)
    swiglu_bwd(ds, h13[..., :F], h13[..., F:], dh13[..., :F], dh13[..., F:])
    return (dh13, swiglu_packed_fwd(h13)) if with_s else dh13


@register("gelu_fwd_out", "eager")
def gelu_fwd_out(x, out=None):
    y = _st(torch.nn.functional.gelu(x.float(), approximate="tanh"), x)
    if out is not None:
        out.copy_(y)
        return out
    return y


@register("gelu_bwd", "eager")
def gelu_bwd(dy, x, out=None):
    xf = x.float()
    k0, k1 = 0.7978845608028654, 0.044715
    t = torch.tanh(k0 * (xf + k1 * xf ** 3))
    g = 0.5 * (1 + t) + 0.5 * xf * (1 - t * t) * k0 * (1 + 3 * k1 * xf * xf)
    d = _st(dy.float() * g, x)
    if out is not None:
        out.copy_(d)
        return out
    return d


# ------------------------------------------------------------------ loss / embedding
@register("ce_loss_fwd_bwd", "eager")
def ce_loss_fwd_bwd(logits, targets, total_rows, loss_out=None, accumulate=False):
    """Overwrites ``logits`` with dlogits; returns the summed loss contribution (fp32 scalar tensor)."""
    lf = logits.float()
    keep = (targets >= 0)
    lse = torch.logsumexp(lf, -1)
    tl = lf.gather(1, targets.clamp(min=0).long().unsqueeze(1)).squeeze(1)
    scale = 1.0 / float(total_rows)
    nll = (lse - tl) * keep.float() * scale
    p = torch.exp(lf - lse.unsqueeze(-1))
    p.scatter_add_(1, targets.clamp(min=0).long().unsqueeze(1), -torch.ones_like(p[:, :1]))
    logits.copy_((p * (keep.float() * scale).unsqueeze(-1)).to(logits.dtype))
    s = nll.sum()
    if loss_out is not None:
        loss_out.copy_((loss_out.float() + s if accumulate else s).reshape(loss_out.shape))
        return loss_out
    return s


@register("embed_fwd", "eager")
def embed_fwd(tok, table, out=None, positions=None, pos_table=None):
    y = table[tok.long()]
    if pos_table is not None:
        y = _st(y.float() + pos_table[positions.long()].float(), table)
    if out is not None:
        out.copy_(y)
        return out
    return y


@register("embed_bwd_accum", "eager")
def embed_bwd_accum(tok, dy, dtable, accumulate=False):
    acc = torch.zeros(dtable.shape, dtype=torch.float32, device=dtable.device)
    valid = tok >= 0
    acc.index_add_(0, tok[valid].long(), dy[valid].float())
    if accumulate:
        acc += dtable.float()
        dtable.copy_(acc.to(dtable.dtype))
    else:
        # rows not hit stay zero on a create
        dtable.copy_(acc.to(dtable.dtype))
    return dtable


# ------------------------------------------------------------------ optimizers
@register("adamw_step", "eager")
def adamw_step(w, g, m, v, lr, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.0, step=1, master=None, gscale=1.0):
    gf = g.float() * gscale
    mf = beta1 * m.float() + (1 - beta1) * gf
    vf = beta2 * v.float() + (1 - beta2) * gf * gf
    m.copy_(mf.to(m.dtype))
    v.copy_(vf.to(v.dtype))
    mh = m.float() / (1 - beta1 ** step)
    vh = v.float() / (1 - beta2 ** step)
    src = master if master is not None else w
    wf = src.float()
    wf = wf - lr * (mh / (vh.sqrt() + eps) + wd * wf)
    if master is not None:
        master.copy_(wf)
    w.copy_(wf.to(w.dtype))
    return w


def split_master_join(w, lo):
    """fp32 master from a bf16 weight (high half) and its int16 low-half plane."""
    hi = w.view(torch.int16).to(torch.int32) << 16
    return (hi + lo.view(torch.int16).to(torch.int32)).view(torch.float32)


def split_master_cut(x):
    """fp32 -> (bf16 weight rounded half away from zero, int16 low half); exact inverse of the join."""
    b = x.contiguous().view(torch.int32)
    hi = ((b + 0x8000) >> 16).to(torch.int16).view(torch.bfloat16)
    lo = (b & 0xFFFF).to(torch.int16)
    return hi, lo


@register("adamw_split_step", "eager")
def adamw_split_step(w, lo, g, m, v, lr, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.0, step=1, gscale=1.0):
    gf = g.float() * gscale
    m.copy_((beta1 * m.float() + (1 - beta1) * gf).to(m.dtype))
    v.copy_((beta2 * v.float() + (1 - beta2) * gf * gf).to(v.dtype))
    mh = m.float() / (1 - beta1 ** step)
    vh = v.float() / (1 - beta2 ** step)
    wf = split_master_join(w, lo)
    wf = wf - lr * (mh / (vh.sqrt() + eps) + wd * wf)
    hi, low = split_master_cut(wf)
    w.copy_(hi)
    lo.view(torch.int16).copy_(low)
    return w


@register("sgd_step", "eager")
def sgd_step(w, g, m=None, lr=1e-2, momentum=0.0, wd=0.0):
    gf = g.float()
    if m is not None:
        m.copy_((momentum * m.float() + gf).to(m.dtype))
        gf = m.float()
    w.copy_((w.float() * (1 - lr * wd) - lr * gf).to(w.dtype))
    return w


# ------------------------------------------------------------------ linear triple (W stored (in, out))
def _mm(a, b):
    if a.dtype == torch.float32 or a.device.type == "cpu":
        return a.float() @ b.float()
    return (a @ b).float()


@register("linear_fwd_bf16", "eager")
def linear_fwd(x, w, out=None, add=None, bias=None):
    y = _mm(x, w)
    if bias is not None:
        y = y + bias.float()
    if add is not None:
        y = y + add.float()
    y = y.to(out.dtype if out is not None else x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


@register("linear_dgrad_bf16", "eager")
def linear_dgrad(dy, w, out=None, add=None):
    dx = _mm(dy, w.t())
    if add is not None:
        dx = dx + add.float()
    dx = dx.to(out.dtype if out is not None else dy.dtype)
    if out is not None:
        out.copy_(dx)
        return out
    return dx


@register("linear_wgrad_bf16", "eager")
def linear_wgrad(x, dy, dw, accumulate=False):
    g = _mm(x.t(), dy)
    if accumulate:
        g = g + dw.float()
    dw.copy_(g.to(dw.dtype))
    return dw


@register("bias_grad", "eager")
def bias_grad(dy, db, accumulate=False):
    g = dy.float().reshape(-1, dy.shape[-1]).sum(0)
    if accumulate:
        g = g + db.float()
    db.copy_(g.to(db.dtype))
    return db


@register("add", "eager")
def add(a, b, out=None):
    y = _st(a.float() + b.float(), a)
    if out is not None:
        out.copy_(y)
        return out
    return y


# ------------------------------------------------------------------ mixture of experts (oracle lane)
# Routing math is fp32 from the given logits; ties go to the SMALLEST expert index in every mode.
# Semantics follow the reference's router / dispatch ops (src/dataflow_training/kernels/moe_router.py:42-111,
# kernels/moe_dispatch.py:49-235); the padded expert-major layout below is this repository's own.
MOE_TILE_ROWS = 256          # expert segments are padded to whole GEMM row tiles


def _topk_smallest_index(scores, k):
    """Top-k by value, ties broken towards the smaller index (a stable descending sort)."""
    order = torch.sort(scores, dim=-1, descending=True, stable=True).indices
    ids = order[..., :k]
    return scores.gather(-1, ids), ids


@register("moe_topk_softmax", "eager")
def moe_topk_softmax(logits, top_k: int, mode: str = "topk_then_softmax"):
    z = logits.float()
    if mode == "topk_then_softmax":
        vals, ids = _topk_smallest_index(z, top_k)
        w = torch.softmax(vals, dim=-1)
    elif mode == "softmax_then_topk":
        p = torch.softmax(z, dim=-1)
        w, ids = _topk_smallest_index(p, top_k)
    else:
        raise KeyError(f"routing mode {mode!r}")
    return w, ids.to(torch.int32)


@register("moe_topk_sigmoid_noaux", "eager")
def moe_topk_sigmoid_noaux(logits, bias, top_k: int, n_group: int = 1, topk_group: int = 1, routed_scaling: float = 1.0,
                           norm_topk: bool = True):
    """DeepSeek-V3 routing: sigmoid scores; selection on score + bias restricted to the best ``topk_group`` of
    ``n_group`` expert groups (a group's rank = sum of its two best biased scores); weights from the unbiased
    scores, normalised over the selection and scaled."""
    s = torch.sigmoid(logits.float())
    sel = s + bias.float().unsqueeze(0)
    t, e = s.shape
    if n_group > 1:
        g = sel.view(t, n_group, e // n_group)
        top2 = torch.sort(g, dim=-1, descending=True, stable=True).values[..., :2].sum(-1)
        _, gid = _topk_smallest_index(top2, topk_group)
        mask = torch.zeros(t, n_group, dtype=torch.bool, device=s.device).scatter_(1, gid, True)
        sel = torch.where(mask.unsqueeze(-1).expand_as(g).reshape(t, e), sel, torch.full_like(sel, float("-inf")))
    _, ids = _topk_smallest_index(sel, top_k)
    w = s.gather(1, ids)
    if norm_topk:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * routed_scaling, ids.to(torch.int32)


@register("moe_router_bwd", "eager")
def moe_router_bwd(dprob, route_w, route_ids, logits, mode: str = "topk_then_softmax"):
    """d(logits) (t, E) fp32 from d(route weights) (t, K)."""
    ids = route_ids.long()
    dp = dprob.float()
    out = torch.zeros(logits.shape, dtype=torch.float32, device=logits.device)
    if mode == "topk_then_softmax":
        p = route_w.float()
        out.scatter_(1, ids, p * (dp - (p * dp).sum(-1, keepdim=True)))
    else:
        pf = torch.softmax(logits.float(), dim=-1)
        tp = pf.gather(1, ids)
        out.copy_(-pf * (dp * tp).sum(-1, keepdim=True))
        out.scatter_add_(1, ids, dp * tp)
    return out


@register("moe_aux_lb_grad", "eager")
def moe_aux_lb_grad(logits, counts, dlogits, alpha: float, top_k: int):
    """Adds the load-balance gradient (alpha E / T) p (f - <f, p>) in place; f = counts / (T K) is detached."""
    t, e = logits.shape
    p = torch.softmax(logits.float(), dim=-1)
    f = counts.float() / (t * top_k)
    dlogits.add_((alpha * e / t) * p * (f.unsqueeze(0) - (p @ f).unsqueeze(1)))
    return dlogits


@register("moe_sort", "eager")
def moe_sort(route_ids, n_experts: int, tile_rows: int = MOE_TILE_ROWS):
    """Padded expert-major layout of the t*K routed slots, computed without a host sync.

    Returns ``(row_of (t, K) int32, row_src (Mp,) int32, offsets_pad (E + 1,) int32, tile_expert (Mp / tile,) int32,
    counts (E,) int32)``: slot (t, k) lives in row ``row_of[t, k]`` of the dispatched matrix; ``row_src[r]`` is the
    token a row holds (-1 for padding); expert e owns rows ``[offsets_pad[e], offsets_pad[e + 1])``, a whole number
    of ``tile_rows`` tiles; ``tile_expert`` names the expert of every row tile (-1 past the end).  ``Mp`` is the
    static worst case ``roundup(t K) + E * tile_rows``.  Within an expert rows keep token order (stable)."""
    t, k = route_ids.shape
    n = t * k
    flat = route_ids.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices                         # expert-major, stable
    counts = torch.zeros(n_experts, dtype=torch.int64, device=flat.device).scatter_add_(0, flat, torch.ones_like(flat))
    padded = (counts + tile_rows - 1) // tile_rows * tile_rows
    off = torch.zeros(n_experts + 1, dtype=torch.int64, device=flat.device)
    off[1:] = torch.cumsum(counts, 0)
    off_pad = torch.zeros(n_experts + 1, dtype=torch.int64, device=flat.device)
    off_pad[1:] = torch.cumsum(padded, 0)
    e_sorted = flat[order]
    rank = torch.arange(n, device=flat.device) - off[e_sorted]
    rows = off_pad[e_sorted] + rank                                       # padded row of each sorted slot
    mp = (n + tile_rows - 1) // tile_rows * tile_rows + n_experts * tile_rows
    row_of = torch.empty(n, dtype=torch.int64, device=flat.device)
    row_of[order] = rows
    row_src = torch.full((mp,), -1, dtype=torch.int64, device=flat.device)
    row_src[rows] = order // k
    tiles = torch.arange(mp // tile_rows, device=flat.device) * tile_rows
    tile_expert = torch.searchsorted(off_pad[1:], tiles, right=True)
    tile_expert = torch.where(tiles < off_pad[-1], tile_expert, torch.full_like(tile_expert, -1))
    return (row_of.view(t, k).to(torch.int32), row_src.to(torch.int32), off_pad.to(torch.int32),
            tile_expert.to(torch.int32), counts.to(torch.int32))


@register("moe_dispatch", "eager")
def moe_dispatch(x, row_src, out=None):
    """xp[r] = x[row_src[r]] (zeros where row_src < 0)."""
    src = row_src.long()
    xp = x[src.clamp(min=0)] * (src >= 0).unsqueeze(-1).to(x.dtype)
    if out is not None:
        out.copy_(xp)
        return out
    return xp


@register("moe_combine", "eager")
def moe_combine(base, yp, route_w, row_of, out=None):
    """y[t] = base[t] + sum_k route_w[t, k] * yp[row_of[t, k]]  (fp32 accumulate, one rounding)."""
    t, k = row_of.shape
    g = yp[row_of.reshape(-1).long()].float().view(t, k, -1)
    y = (g * route_w.float().unsqueeze(-1)).sum(1)
    if base is not None:
        y = y + base.float()
    y = y.to(yp.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


@register("moe_dispatch_bwd", "eager")
def moe_dispatch_bwd(dxp, row_of, out=None, accumulate: bool = False):
    """dx[t] (+)= sum_k dxp[row_of[t, k]]."""
    t, k = row_of.shape
    g = dxp[row_of.reshape(-1).long()].float().view(t, k, -1).sum(1)
    if out is None:
        return g.to(dxp.dtype)
    out.copy_((out.float() + g if accumulate else g).to(out.dtype))
    return out


@register("moe_scale_rows", "eager")
def moe_scale_rows(xp, route_w, row_of):
    """In place: row row_of[t, k] of xp is multiplied by route_w[t, k] (padding rows untouched)."""
    idx = row_of.reshape(-1).long()
    xp[idx] = (xp[idx].float() * route_w.reshape(-1, 1).float()).to(xp.dtype)
    return xp


@register("moe_rowdot", "eager")
def moe_rowdot(a, b, row_of):
    """(t, K) fp32: <a[row], b[row]> for row = row_of[t, k]."""
    idx = row_of.reshape(-1).long()
    return (a[idx].float() * b[idx].float()).sum(-1).view(row_of.shape)


@register("moe_grouped_mm", "eager")
def moe_grouped_mm(xp, w, tile_expert, out=None, transpose_w: bool = False):
    """Rows of expert e times ``w[e]`` ((K, N), or its transpose): (Mp, K) -> (Mp, N).  ``tile_expert`` names the expert
    of every ``MOE_TILE_ROWS`` row tile (-1: no expert, rows stay zero).  Padding rows are zero in, zero out."""
    n = w.shape[1] if transpose_w else w.shape[2]
    y = out if out is not None else torch.zeros(xp.shape[0], n, dtype=xp.dtype, device=xp.device)
    if out is not None:
        y.zero_()
    te = tile_expert.tolist()
    tile = xp.shape[0] // max(len(te), 1) if len(te) * MOE_TILE_ROWS != xp.shape[0] else MOE_TILE_ROWS
    i = 0
    while i < len(te):
        j = i
        while j < len(te) and te[j] == te[i]:
            j += 1
        if te[i] >= 0:
            wi = w[te[i]].t() if transpose_w else w[te[i]]
            y[i * tile:j * tile] = _mm(xp[i * tile:j * tile], wi).to(y.dtype)
        i = j
    return y


@register("moe_grouped_wgrad", "eager")
def moe_grouped_wgrad(xp, dyp, offsets_pad, dw, accumulate: bool = False):
    """dw[e] (+)= xp_e^T dyp_e."""
    off = offsets_pad.tolist() if offsets_pad.device.type == "cpu" else offsets_pad.cpu().tolist()
    for i in range(dw.shape[0]):
        a, b = off[i], off[i + 1]
        g = _mm(xp[a:b].t(), dyp[a:b]) if b > a else torch.zeros_like(dw[i], dtype=torch.float32)
        dw[i].copy_((dw[i].float() + g.float() if accumulate else g).to(dw.dtype))
    return dw


# ------------------------------------------------------------------ sparse-attention indexer
@register("dsa_index_scores", "eager")
def dsa_index_scores(q, k, wgt, seg_start, q0: int, q1: int, key_lo: int):
    """I[i, j] = sum_h wgt[i, h] * relu(<q[i, h], k[j]>) for query rows [q0, q1) against keys [key_lo, q1); -inf where query i
    does not see key j (another sequence, or j > i).  q (n, H, D), k (n, D), wgt (n, H) fp32, seg_start (n,) int: the first
    row of every row's sequence.  Returns (q1 - q0, q1 - key_lo) fp32."""
    s = torch.relu(torch.einsum("ihd,jd->ihj", q[q0:q1].float(), k[key_lo:q1].float()))
    s = (s * wgt[q0:q1].float()[:, :, None]).sum(1)
    rows = torch.arange(q0, q1, device=q.device)[:, None]
    cols = torch.arange(key_lo, q1, device=q.device)[None, :]
    return s.masked_fill(~((cols <= rows) & (cols >= seg_start[q0:q1].long()[:, None])), float("-inf"))


@register("dsa_topk_rows", "eager")
def dsa_topk_rows(scores, k: int, col_base: int = 0):
    """The k largest entries of every row as ASCENDING key indices (+ col_base); ties go to the smaller index; -1 where a row
    has fewer than k finite entries.  Returns (rows, k) int32."""
    rows, cols = scores.shape
    kk = min(k, cols)
    # a stable sort by descending value keeps equal values in index order
    order = torch.sort(scores, dim=1, descending=True, stable=True).indices[:, :kk]
    vals = scores.gather(1, order)
    idx = torch.where(vals > float("-inf"), order, torch.full_like(order, cols))
    idx = torch.sort(idx, dim=1).values
    idx = torch.where(idx >= cols, torch.full_like(idx, -1), idx + col_base)
    # dead slots stay where the ascending order puts them: at the end
    if kk < k:
        idx = torch.nn.functional.pad(idx, (0, k - kk), value=-1)
    return idx.to(torch.int32)


# ------------------------------------------------------------------ sequence-mixing helpers (linear / latent attention families)
@register("l2norm_fwd", "eager")
def l2norm_fwd(x, eps: float = 1e-6):
    """y = x * rsqrt(sum x^2 + eps) over the last dim.  Returns (y, rstd (rows,) fp32)."""
    r = torch.rsqrt(x.float().pow(2).sum(-1) + eps)
    return (x.float() * r.unsqueeze(-1)).to(x.dtype), r.reshape(-1)


@register("l2norm_bwd", "eager")
def l2norm_bwd(dy, x, rstd):
    r = rstd.reshape(*x.shape[:-1], 1)
    xf, gf = x.float(), dy.float()
    return (r * gf - xf * r.pow(3) * (xf * gf).sum(-1, keepdim=True)).to(x.dtype)


@register("gated_rmsnorm_fwd", "eager")
def gated_rmsnorm_fwd(x, g, w, eps: float = 1e-6):
    """y = rmsnorm(x) * w * silu(g).  Returns (y, rstd (rows,) fp32)."""
    r = torch.rsqrt(x.float().pow(2).mean(-1) + eps)
    n = (x.float() * r.unsqueeze(-1)).to(x.dtype) * w
    return n * torch.nn.functional.silu(g.float()).to(x.dtype), r.reshape(-1)


@register("gated_rmsnorm_bwd", "eager")
def gated_rmsnorm_bwd(dy, x, g, w, rstd):
    """Returns (dx, dg, dw fp32)."""
    r = rstd.reshape(*x.shape[:-1], 1)
    xf, gf, gy, wf = x.float(), g.float(), dy.float(), w.float()
    sg = torch.sigmoid(gf)
    nrm = xf * r
    dg = gy * nrm * wf * (sg * (1 + gf * (1 - sg)))
    d_n = gy * gf * sg
    dw = (d_n * nrm).reshape(-1, x.shape[-1]).sum(0)
    dn = d_n * wf
    dx = r * dn - xf * r.pow(3) * (dn * xf).mean(-1, keepdim=True)
    return dx.to(x.dtype), dg.to(x.dtype), dw


@register("conv_silu_fwd", "eager")
def conv_silu_fwd(x, w, seg_start):
    """Depthwise causal convolution along tokens (width w.shape[1]) that never crosses a segment start, then SiLU."""
    n, width = x.shape[0], w.shape[1]
    idx = torch.arange(n, device=x.device)
    acc = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    for j in range(width):
        src = idx - (width - 1 - j)
        ok = (src >= seg_start.long()).float()[:, None]
        acc = acc + x[src.clamp(min=0)].float() * ok * w[:, j].float()[None, :]
    return torch.nn.functional.silu(acc.to(x.dtype).float()).to(x.dtype)


@register("conv_silu_bwd", "eager")
def conv_silu_bwd(dy, x, w, seg_start):
    """Returns (dx, dw fp32) by differentiating the forward."""
    with torch.enable_grad():
        xf, wf = x.float().detach().requires_grad_(True), w.float().detach().requires_grad_(True)
        n, width = x.shape[0], w.shape[1]
        idx = torch.arange(n, device=x.device)
        acc = 0
        for j in range(width):
            src = idx - (width - 1 - j)
            acc = acc + xf[src.clamp(min=0)] * (src >= seg_start.long()).float()[:, None] * wf[:, j][None, :]
        y = torch.nn.functional.silu(acc)
        gx, gw = torch.autograd.grad(y, [xf, wf], dy.float())
    return gx.to(x.dtype), gw


# ------------------------------------------------------------------ fp8 lane (row-wise e4m3 scales)
FP8_MAX = 448.0


@register("quant_fp8_rowwise", "eager")
def quant_fp8_rowwise(x):
    """x (rows, K) -> (q (rows, K) float8_e4m3fn, scale (rows,) fp32) with x ~= q * scale[:, None]."""
    amax = x.float().abs().amax(-1)
    scale = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (x.float() / scale[:, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale


@register("linear_fwd_fp8", "eager")
def linear_fwd_fp8(x, w, out=None, add=None, bias=None):
    """``linear_fwd_bf16`` with both operands rounded to e4m3 first: x (M, K) per row, w (K, N) stored (in, out) per output
    column; fp32 accumulation, scales applied to the accumulator, one rounding to the output dtype."""
    xq, sx = quant_fp8_rowwise(x)
    wq, sw = quant_fp8_rowwise(w.t().contiguous())
    return linear_fp8(xq, sx, wq, sw, out=out, add=add, bias=bias, out_dtype=out.dtype if out is not None else x.dtype)


@register("linear_fp8", "eager")
def linear_fp8(xq, x_scale, wq, w_scale, out=None, add=None, bias=None, out_dtype=torch.bfloat16):
    """y (M, N) = (xq * x_scale[:, None]) @ (wq * w_scale[:, None])^T (+ bias) (+ add); wq stored (N, K)."""
    y = (xq.float() @ wq.float().t()) * x_scale[:, None] * w_scale[None, :]
    if bias is not None:
        y = y + bias.float()
    if add is not None:
        y = y + add.float()
    y = y.to(out_dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y
