"""Reference forms, in differentiable torch, of the inner ops the newer families share: RMSNorm, rotate-half RoPE on a
slice, causal segment masks, SwiGLU, a mixture-of-experts MLP with either softmax or sigmoid "no-aux" grouped routing
and optional shared experts, multi-head latent attention, the sparse-attention indexer, and the gated delta rule.
Reference role: ``src/dataflow_training/blocks/modules/{mla_forms,dsa_forms}.py``, ``moe/forms.py`` and the DeltaNet
references of ``blocks/ops.py:509-623``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def rmsnorm(x, w, eps: float):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def rope(x, positions, theta: float):
    """Rotate-half RoPE over the last dim of x (tokens, heads, dim)."""
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    cos, sin = torch.cos(ang)[:, None, :].to(x.dtype), torch.sin(ang)[:, None, :].to(x.dtype)
    x1, x2 = x[..., :d // 2], x[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def segment_causal_mask(seg, n: int, device):
    """(n, n) bool: query i may see key j (same segment, j <= i)."""
    pos = seg.positions.to(device)[:n].long()
    idx = torch.arange(n, device=device)
    start = idx - pos                                     # first token of the segment each token lives in
    return (start[:, None] == start[None, :]) & (idx[None, :] <= idx[:, None])


def attention(q, k, v, mask, scale: float):
    """q (n, h, dq), k (n, hk, dq), v (n, hk, dv); grouped heads; ``mask`` (n, n) or (h, n, n) bool."""
    h, hk = q.shape[1], k.shape[1]
    if hk != h:
        k, v = k.repeat_interleave(h // hk, 1), v.repeat_interleave(h // hk, 1)
    s = torch.einsum("ihd,jhd->hij", q.float(), k.float()) * scale
    s = s.masked_fill(~(mask if mask.dim() == 3 else mask[None]), float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, v.float()).to(q.dtype), p


class _LinearFp8(torch.autograd.Function):
    """y = x @ w with both operands rounded to e4m3 (per-row scales for x, per-output-column scales for w, fp32
    accumulation) in the forward; the backward products run in the storage dtype on the unquantised operands."""

    @staticmethod
    def forward(ctx, x, w):
        from ..ops import resolve_kernels
        ks = _native(x) or resolve_kernels(kernel_set="eager")
        ctx.save_for_backward(x, w)
        return ks.linear_fwd_fp8(x.contiguous(), w.contiguous())

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        return dy @ w.t(), x.t() @ dy


def linear(x, w, precision: str = "bf16"):
    """x (n, k) @ w (k, m); ``precision="fp8"``: e4m3 operands in the forward (see ``ops`` ``linear_fwd_fp8``)."""
    if precision == "fp8" and x.dim() == 2 and x.shape[1] % 16 == 0 and w.shape[1] % 16 == 0:
        return _LinearFp8.apply(x, w)
    return x @ w


def swiglu_mlp(x, w13, w2, precision: str = "bf16"):
    h = linear(x, w13, precision)
    f = h.shape[-1] // 2
    return linear(F.silu(h[..., :f].float()).to(x.dtype) * h[..., f:], w2, precision)


def route_softmax_topk(logits, k: int):
    vals, ids = torch.topk(logits.float(), k, dim=-1)
    return torch.softmax(vals, -1), ids


def route_sigmoid_noaux(logits, bias, k: int, n_group: int, topk_group: int, scaling: float):
    """Sigmoid scores; selection on score + bias inside the best ``topk_group`` of ``n_group`` expert groups (a group's
    rank is the sum of its two best biased scores); weights from the unbiased scores, normalised and scaled."""
    K = _native(logits)
    if K is not None and logits.shape[1] <= 256 and k <= 16:
        # selection by the native router; the weights are re-derived from the scores so that gradients reach the router
        _, ids = K.moe_topk_sigmoid_noaux(logits.detach(), bias, k, n_group, topk_group, scaling)
        w = torch.sigmoid(logits.float()).gather(1, ids.long())
        return w / (w.sum(-1, keepdim=True) + 1e-20) * scaling, ids.long()
    s = torch.sigmoid(logits.float())
    sel = s + bias.float()[None]
    t, e = s.shape
    if n_group > 1:
        g = sel.view(t, n_group, e // n_group)
        rank = g.topk(min(2, e // n_group), dim=-1).values.sum(-1)
        keep = torch.zeros_like(rank, dtype=torch.bool).scatter_(1, rank.topk(topk_group, dim=-1).indices, True)
        sel = sel.masked_fill(~keep[:, :, None].expand_as(g).reshape(t, e), float("-inf"))
    ids = sel.topk(k, dim=-1).indices
    w = s.gather(1, ids)
    return w / (w.sum(-1, keepdim=True) + 1e-20) * scaling, ids


def moe_mlp(x, w13_experts, w2_experts, weights, ids):
    """Token-choice experts, dense loop over experts (reference form)."""
    y = torch.zeros_like(x)
    for e in range(w13_experts.shape[0]):
        tok, slot = (ids == e).nonzero(as_tuple=True)
        if tok.numel():
            y = y.index_add(0, tok, swiglu_mlp(x[tok], w13_experts[e], w2_experts[e]) * weights[tok, slot].to(x.dtype)[:, None])
    return y


class _EpMoE(torch.autograd.Function):
    """Routed experts with the experts split over the ranks of an expert-parallel group: the forward is dispatch +
    grouped up-projection, SwiGLU, grouped down-projection + weighted combine (``parallel/ep.py``), the backward the same
    two exchanges with the roles of the matrices swapped.  Every rank calls it at the same point of its program."""

    @staticmethod
    def forward(ctx, x, w13, w2, weights, ids, group):
        from ..parallel.ep import ep_moe_forward
        y, saved = ep_moe_forward(group, x.contiguous(), ids.to(torch.int32).contiguous(), weights.float().contiguous(), w13, w2)
        ctx.group, ctx.kept, ctx.wdtype = group, saved, weights.dtype
        ctx.save_for_backward(w13, w2)
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..parallel.ep import ep_moe_backward
        w13, w2 = ctx.saved_tensors
        dw13, dw2 = torch.zeros_like(w13), torch.zeros_like(w2)
        dh, dwts = ep_moe_backward(ctx.group, dy.contiguous(), ctx.kept, w13, w2, dw13, dw2, accumulate=False)
        return dh, dw13, dw2, dwts.to(ctx.wdtype), None, None


def moe_mlp_ep(x, w13_local, w2_local, weights, ids, group):
    """``moe_mlp`` when this rank holds ``E / world`` of the experts (``w13_local`` (E_local, d, 2F)); ``ids`` name
    experts of the whole model."""
    return _EpMoE.apply(x, w13_local, w2_local, weights, ids, group)


def load_balance_aux(logits, ids, coef: float):
    """Switch-style balance loss coef * E * sum_e f_e * p_e (f: fraction of slots, p: mean router probability)."""
    if not coef:
        return None
    t, e = logits.shape
    p = torch.softmax(logits.float(), -1).mean(0)
    f = torch.zeros(e, device=logits.device).scatter_add_(0, ids.reshape(-1), torch.ones(ids.numel(), device=logits.device)) / ids.numel()
    return coef * e * (f.detach() * p).sum() * t


def mla_qkv(x, w, cfg, positions):
    """Multi-head latent attention projections: two low-rank stacks, decoupled RoPE with one shared rope key.
    Returns q (n, h, nope + rope), k (n, h, nope + rope), v (n, h, dv) and the normalised q latent (``x`` itself when the
    query has no low-rank stack), which is what the sparse-attention indexer reads."""
    n, h = x.shape[0], cfg.n_heads
    if cfg.q_lora:
        cq = rmsnorm(x @ w["wq_a"], w["q_norm"], cfg.rms_eps)
        q = (cq @ w["wq_b"]).view(n, h, cfg.d_nope + cfg.d_rope)
    else:
        cq = x
        q = (x @ w["wq"]).view(n, h, cfg.d_nope + cfg.d_rope)
    kv_a = x @ w["wkv_a"]                                           # (n, kv_lora + rope)
    ckv = rmsnorm(kv_a[:, :cfg.kv_lora], w["kv_norm"], cfg.rms_eps)
    k_rope = rope(kv_a[:, None, cfg.kv_lora:], positions, cfg.rope_theta)              # (n, 1, rope): shared by the heads
    kv = (ckv @ w["wkv_b"]).view(n, h, cfg.d_nope + cfg.d_v)
    q = torch.cat([q[..., :cfg.d_nope], rope(q[..., cfg.d_nope:], positions, cfg.rope_theta)], -1)
    k = torch.cat([kv[..., :cfg.d_nope], k_rope.expand(n, h, cfg.d_rope)], -1)
    return q, k, kv[..., cfg.d_nope:], cq


def _rope_first(t, positions, cfg):
    """Rotate the first ``d_rope`` dims of the last axis, leave the rest (the indexer's rope-first layout)."""
    r = min(cfg.d_rope, t.shape[-1])
    return torch.cat([rope(t[..., :r], positions, cfg.rope_theta), t[..., r:]], -1) if r else t


def dsa_index_scores(x, cq, w, cfg, positions, ln_eps: float = 1e-5):
    """Lightning indexer: I[i, j] = sum_h wgt[i, h] * relu(<q_idx[i, h], k_idx[j]>), a few small heads, one shared key.
    Queries come from the normalised q latent ``cq``, the key from ``x`` through a LayerNorm (gain and bias), both rotated
    on their first ``d_rope`` dims only; the head weights wgt = (x w_w) * heads^-1/2 * dim^-1/2; everything in fp32.
    Form parity: reference ``src/dataflow_training/blocks/modules/dsa_forms.py:47-110``."""
    n = x.shape[0]
    qi = _rope_first((cq @ w["wi_q"]).view(n, cfg.index_heads, cfg.index_dim), positions, cfg).float()
    ki = F.layer_norm((x @ w["wi_k"]).float(), (cfg.index_dim,), w["wi_k_gain"].float(), w["wi_k_bias"].float(), ln_eps)
    ki = _rope_first(ki.view(n, 1, cfg.index_dim), positions, cfg)[:, 0].float()
    wgt = (x.float() @ w["wi_w"].float()) * cfg.index_heads ** -0.5 * cfg.index_dim ** -0.5
    s = torch.relu(torch.einsum("ihd,jd->ihj", qi, ki))
    return (s * wgt[:, :, None]).sum(1)


def dsa_topk_mask(scores, causal, k: int):
    """(n, n) bool: the ``k`` best visible keys of every query (all visible keys when there are fewer)."""
    s = scores.masked_fill(~causal, float("-inf"))
    kk = min(k, s.shape[-1])
    idx = s.topk(kk, dim=-1).indices
    return torch.zeros_like(causal).scatter_(1, idx, True) & causal


def mla_latents(x, w, cfg, positions):
    """The inputs of the latent ("absorbed") form of multi-head latent attention: q (n, h, nope + rope) rotated, the
    normalised kv latent (n, kv_lora), the rotated shared rope key (n, rope) and the normalised q latent."""
    n, h = x.shape[0], cfg.n_heads
    if cfg.q_lora:
        cq = rmsnorm(x @ w["wq_a"], w["q_norm"], cfg.rms_eps)
        q = (cq @ w["wq_b"]).view(n, h, cfg.d_nope + cfg.d_rope)
    else:
        cq = x
        q = (x @ w["wq"]).view(n, h, cfg.d_nope + cfg.d_rope)
    kv_a = x @ w["wkv_a"]
    ckv = rmsnorm(kv_a[:, :cfg.kv_lora], w["kv_norm"], cfg.rms_eps)
    k_rope = rope(kv_a[:, None, cfg.kv_lora:], positions, cfg.rope_theta)[:, 0]
    q = torch.cat([q[..., :cfg.d_nope], rope(q[..., cfg.d_nope:], positions, cfg.rope_theta)], -1)
    return q, ckv, k_rope, cq


def _indexer_inputs(x, cq, w, cfg, positions):
    n = x.shape[0]
    qi = _rope_first((cq @ w["wi_q"]).view(n, cfg.index_heads, cfg.index_dim), positions, cfg).float()
    ki = F.layer_norm((x @ w["wi_k"]).float(), (cfg.index_dim,), w["wi_k_gain"].float(), w["wi_k_bias"].float(), 1e-5)
    ki = _rope_first(ki.view(n, 1, cfg.index_dim), positions, cfg)[:, 0].float()
    wgt = (x.float() @ w["wi_w"].float()) * cfg.index_heads ** -0.5 * cfg.index_dim ** -0.5
    return qi, ki, wgt


def dsa_select(x, cq, w, cfg, positions, k: int, chunk: int = 256):
    """Top-``k`` visible keys of every query WITHOUT the (n, n) score matrix: index scores are formed for ``chunk`` queries at
    a time against the keys up to the chunk's end, and only the selection leaves.  Returns ``sel`` (n, kk) int64 key rows and
    ``live`` (n, kk) bool — false where a query sees fewer than kk keys (those slots name arbitrary rows).  No gradient.
    Role parity: reference ``src/dataflow_training/kernels/dsa.py`` (index scores + top-k)."""
    n = x.shape[0]
    with torch.no_grad():
        qi, ki, wgt = _indexer_inputs(x, cq, w, cfg, positions)
        idx = torch.arange(n, device=x.device)
        start = idx - positions[:n].long()
        kk = min(k, n)
        K = _native(x)
        if K is not None and cfg.index_dim in (64, 128) and "dsa_index_scores" in K.native_ops():
            # device kernels: scores of 1024 queries at a time on the tensor cores, then a deterministic row selection
            qb, kb, st = qi.to(torch.bfloat16).contiguous(), ki.to(torch.bfloat16).contiguous(), start.to(torch.int32)
            rows = []
            for a in range(0, n, 1024):
                b = min(a + 1024, n)
                rows.append(K.dsa_topk_rows(K.dsa_index_scores(qb, kb, wgt, st, a, b, 0), kk, 0))
            got = torch.cat(rows).long()
            return got.clamp(min=0), got >= 0
        sel = torch.empty(n, kk, dtype=torch.long, device=x.device)
        live = torch.empty(n, kk, dtype=torch.bool, device=x.device)
        for a in range(0, n, chunk):
            b = min(a + chunk, n)
            lo = int(start[a])                                   # the earliest sequence start any query of the chunk sees
            s = torch.relu(torch.einsum("ihd,jd->ihj", qi[a:b], ki[lo:b]))
            s = (s * wgt[a:b, :, None]).sum(1)                   # (chunk, keys lo..b)
            cols = idx[lo:b]
            vis = (cols[None, :] <= idx[a:b, None]) & (cols[None, :] >= start[a:b, None])
            s = s.masked_fill(~vis, float("-inf"))
            if s.shape[1] < kk:
                s = torch.nn.functional.pad(s, (0, kk - s.shape[1]), value=float("-inf"))
            top = s.topk(kk, dim=-1)
            live[a:b] = top.values > float("-inf")
            sel[a:b] = (top.indices + lo).clamp(max=n - 1)
    return sel, live


def dsa_scores_at(x, cq, w, cfg, positions, sel):
    """Index scores at the selected keys only, (n, kk), differentiable with respect to the indexer's fields."""
    qi, ki, wgt = _indexer_inputs(x, cq, w, cfg, positions)
    s = torch.relu(torch.einsum("ihd,ikd->ihk", qi, ki[sel]))
    return (s * wgt[:, :, None]).sum(1)


def dsa_indexer_kl_selected(x, cq, w, cfg, positions, sel, live, target, chunk: int = 512):
    """KL(target || softmax of the index scores over the selection), mean over queries, without the (n, heads, kk) scores of
    the whole round in memory: queries go ``chunk`` at a time and every chunk is re-run in the backward.  Equals
    ``dsa_indexer_kl_at(dsa_scores_at(...), target, live)``."""
    from torch.utils.checkpoint import checkpoint
    n = x.shape[0]
    qi, ki, wgt = _indexer_inputs(x, cq, w, cfg, positions)
    if n <= chunk:
        s = (torch.relu(torch.einsum("ihd,ikd->ihk", qi, ki[sel])) * wgt[:, :, None]).sum(1)
        return dsa_indexer_kl_at(s, target, live)

    def part(qc, wc, selc, livec, tc, ki_):
        s = (torch.relu(torch.einsum("ihd,ikd->ihk", qc, ki_[selc])) * wc[:, :, None]).sum(1)
        logq = torch.log_softmax(s.masked_fill(~livec, float("-inf")), dim=-1)
        term = torch.where(tc > 0, tc * (torch.log(tc.clamp_min(1e-20)) - logq.masked_fill(~livec, 0.0)), torch.zeros_like(tc))
        return term.sum()

    total = x.new_zeros((), dtype=torch.float32)
    for a in range(0, n, chunk):
        b = min(a + chunk, n)
        args = (qi[a:b], wgt[a:b], sel[a:b], live[a:b], target[a:b], ki)
        total = total + (checkpoint(part, *args, use_reentrant=False) if torch.is_grad_enabled() else part(*args))
    return total / n


def mla_sparse_attention(q, ckv, k_rope, wkv_b, sel, live, cfg, chunk: int = 256, want_target: bool = False):
    """Attention of every query over ITS selected keys in the latent form: with k_j = [W_kb^T c_j | r_j] and
    v_j = W_vb^T c_j, the logits are (W_kb q_nope) . c_j + q_rope . r_j and the output is W_vb^T (sum_j p_j c_j) — one
    gathered (kk, kv_lora + rope) block per query serves every head, and nothing of size (n, n) exists.  Queries are
    processed ``chunk`` at a time (each chunk re-run in the backward).  Returns (n, h, dv) and, when asked, the
    head-summed probabilities at the selection (n, kk), detached.
    Role parity: reference ``src/dataflow_training/kernels/dsa.py`` (sparse attention forward / backward)."""
    from torch.utils.checkpoint import checkpoint
    n, h = q.shape[0], cfg.n_heads
    wb = wkv_b.view(cfg.kv_lora, h, cfg.d_nope + cfg.d_v)
    w_kb, w_vb = wb[..., :cfg.d_nope], wb[..., cfg.d_nope:]
    scale = (cfg.d_nope + cfg.d_rope) ** -0.5

    # products in the storage dtype on a device (bf16 tensor cores, fp32 accumulation), softmax in fp32; fp32 inputs stay fp32
    cd = q.dtype if q.is_cuda else torch.float32

    def part(qc, selc, livec, ckv_, kr_, w_kb_, w_vb_):
        q_abs = torch.einsum("ihd,chd->ihc", qc[..., :cfg.d_nope].to(cd), w_kb_.to(cd))            # (c, h, kv_lora)
        kc, kr = ckv_[selc].to(cd), kr_[selc].to(cd)                                                 # (c, kk, kv_lora / rope)
        s = (torch.einsum("ihc,ikc->ihk", q_abs, kc) + torch.einsum("ihr,ikr->ihk", qc[..., cfg.d_nope:].to(cd), kr)).float() * scale
        p = torch.softmax(s.masked_fill(~livec[:, None, :], float("-inf")), dim=-1)
        o = torch.einsum("ihc,chd->ihd", torch.einsum("ihk,ikc->ihc", p.to(cd), kc), w_vb_.to(cd))
        return o.to(qc.dtype), p.detach().sum(1)

    outs, targets = [], []
    for a in range(0, n, chunk):
        b = min(a + chunk, n)
        args = (q[a:b], sel[a:b], live[a:b], ckv, k_rope, w_kb, w_vb)
        o, t = checkpoint(part, *args, use_reentrant=False) if torch.is_grad_enabled() and n > chunk else part(*args)
        outs.append(o)
        targets.append(t)
    out = torch.cat(outs)
    if not want_target:
        return out, None
    t = torch.cat(targets)
    return out, t / (t.sum(-1, keepdim=True) + 1e-20)


def dsa_indexer_kl_at(scores_sel, target_sel, live):
    """``dsa_indexer_kl_to`` on (n, kk) tensors that hold the selected keys only."""
    logq = torch.log_softmax(scores_sel.masked_fill(~live, float("-inf")), dim=-1)
    term = torch.where(target_sel > 0, target_sel * (torch.log(target_sel.clamp_min(1e-20)) - logq.masked_fill(~live, 0.0)),
                       torch.zeros_like(target_sel))
    return term.sum(-1).mean()


def dsa_attention_target(probs):
    """The indexer's training target of one layer: attention probabilities summed over heads, L1-normalised per query,
    detached.  probs (heads, n, n) -> (n, n)."""
    target = probs.detach().sum(0)
    return target / (target.sum(-1, keepdim=True) + 1e-20)


def dsa_indexer_kl_to(scores, target, live):
    """KL(target || softmax of the index scores over the live set), mean over queries; ``target`` is a constant and ``live``
    the keys a query attends to (its selection; the whole causal prefix during the dense warm-up)."""
    logq = torch.log_softmax(scores.masked_fill(~live, float("-inf")), dim=-1)
    term = torch.where(target > 0, target * (torch.log(target.clamp_min(1e-20)) - logq.masked_fill(~live, 0.0)), torch.zeros_like(target))
    return term.sum(-1).mean()


def dsa_indexer_kl(scores, probs, causal):
    """KL(attention distribution summed over heads || softmax of the index scores), mean over queries; the attention
    side is a constant target."""
    return dsa_indexer_kl_to(scores, dsa_attention_target(probs), causal)


_KS = {}


def _native(x):
    """The hand-written kernels, when ``x`` is a bf16 tensor on a device that has them (else ``None``)."""
    if not (x.is_cuda and x.dtype == torch.bfloat16):
        return None
    if "ks" not in _KS:
        from ..ops import resolve_kernels
        ks = resolve_kernels()
        _KS["ks"] = ks if "l2norm_fwd" in ks.native_ops() else None
    return _KS["ks"]


class _L2Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps, K):
        y, rstd = K.l2norm_fwd(x, eps)
        ctx.save_for_backward(x, rstd)
        ctx.K = K
        return y

    @staticmethod
    def backward(ctx, dy):
        x, rstd = ctx.saved_tensors
        return ctx.K.l2norm_bwd(dy, x, rstd), None, None


class _GatedRmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, g, w, eps, K):
        y, rstd = K.gated_rmsnorm_fwd(x, g, w, eps)
        ctx.save_for_backward(x, g, w, rstd)
        ctx.K = K
        return y

    @staticmethod
    def backward(ctx, dy):
        x, g, w, rstd = ctx.saved_tensors
        dx, dg, dw = ctx.K.gated_rmsnorm_bwd(dy, x, g, w, rstd)
        return dx, dg, dw.to(w.dtype), None, None


class _ConvSilu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, seg_start, K):
        ctx.save_for_backward(x, w, seg_start)
        ctx.K = K
        return K.conv_silu_fwd(x, w, seg_start)

    @staticmethod
    def backward(ctx, dy):
        x, w, seg_start = ctx.saved_tensors
        dx, dw = ctx.K.conv_silu_bwd(dy, x, w, seg_start)
        return dx, dw.to(w.dtype), None, None


def l2norm(x, eps: float = 1e-6):
    K = _native(x)
    if K is not None and x.shape[-1] <= 512:
        return _L2Norm.apply(x, eps, K)
    return x * torch.rsqrt(x.float().pow(2).sum(-1, keepdim=True) + eps).to(x.dtype)


def gated_rmsnorm(x, g, w, eps: float):
    """rmsnorm(x) * w * silu(g)."""
    K = _native(x)
    if K is not None and x.shape[-1] <= 512:
        return _GatedRmsNorm.apply(x, g.to(x.dtype), w, eps, K)
    return rmsnorm(x, w, eps) * F.silu(g.float()).to(x.dtype)


def causal_conv1d_silu(x, w, seg_start):
    """Depthwise causal convolution of width ``w.shape[1]`` along tokens, never crossing a segment start, then SiLU.
    x (n, c), w (c, width), seg_start (n,) index of the first token of each token's segment."""
    K = _native(x)
    if K is not None and w.shape[1] <= 4:
        return _ConvSilu.apply(x, w, seg_start.to(torch.int32), K)
    n, width = x.shape[0], w.shape[1]
    idx = torch.arange(n, device=x.device)
    out = torch.zeros_like(x)
    for j in range(width):
        src = idx - (width - 1 - j)
        ok = (src >= seg_start).to(x.dtype)[:, None]
        out = out + x[src.clamp(min=0)] * ok * w[:, j][None, :]
    return F.silu(out.float()).to(x.dtype)


def gated_delta_rule_sequential(q, k, v, g, beta, seg_start):
    """Sequential form, one token at a time (the oracle of the chunked form below):
    S <- exp(g_t) S (I - beta_t k_t k_t^T) + beta_t v_t k_t^T;  o_t = S q_t.
    q, k (n, h, dk) l2-normalised; v (n, h, dv); g (n, h) log-decay <= 0; beta (n, h) in (0, 1).  State resets at
    segment starts."""
    n, h, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(h, dv, dk, dtype=torch.float32, device=q.device)
    outs = []
    qf, kf, vf = q.float() * dk ** -0.5, k.float(), v.float()
    for t in range(n):
        if int(seg_start[t]) == t:
            S = torch.zeros_like(S)
        S = S * torch.exp(g[t].float())[:, None, None]
        kt, vt, bt = kf[t], vf[t], beta[t].float()[:, None]
        pred = torch.einsum("hvk,hk->hv", S, kt)
        S = S + torch.einsum("hv,hk->hvk", bt * (vt - pred), kt)
        outs.append(torch.einsum("hvk,hk->hv", S, qf[t]))
    return torch.stack(outs, 0).to(q.dtype)


def _delta_rule_chunks(q, k, v, g, beta, chunk: int):
    """The chunk-parallel form over a batch of equal-length sequences.  q, k (b, L, h, dk), v (b, L, h, dv), g / beta (b, L, h),
    fp32, L a multiple of ``chunk`` (padding rows carry beta = 0, g = 0: they change nothing).  Returns o (b, L, h, dv).

    Inside a chunk with state S0 at its start, cumulative decay G_t = sum_{i <= t} g_i and pseudo-values u_t defined by
    S_t = exp(g_t) S_{t-1} + u_t k_t^T, the recurrence unrolls to a triangular system (the WY form of the delta rule):
        (I + diag(beta) L) U = diag(beta) (V - (exp(G) * K) S0^T),   L[t, s] = exp(G_t - G_s) (k_t . k_s) for s < t
        O = (exp(G) * Q) S0^T + (A * mask_{s <= t}) U,                A[t, s] = exp(G_t - G_s) (q_t . k_s)
        S_end = exp(G_end) S0 + U^T (exp(G_end - G) * K)
    so a chunk costs a handful of matrix products and one triangular solve, and only S crosses chunk borders."""
    b, L, h, dk = q.shape
    dv = v.shape[-1]
    C = chunk
    nc = L // C
    # (b, h, nc, C, d): heads become a batch axis of the matrix products
    qc = q.permute(0, 2, 1, 3).reshape(b, h, nc, C, dk)
    kc = k.permute(0, 2, 1, 3).reshape(b, h, nc, C, dk)
    vc = v.permute(0, 2, 1, 3).reshape(b, h, nc, C, dv)
    gc = g.permute(0, 2, 1).reshape(b, h, nc, C)
    bc = beta.permute(0, 2, 1).reshape(b, h, nc, C)
    G = gc.cumsum(-1)                                                    # (b, h, nc, C), <= 0 and non-increasing
    diff = G[..., :, None] - G[..., None, :]                             # G_t - G_s
    idx = torch.arange(C, device=q.device)
    lower = idx[:, None] > idx[None, :]
    lower_eq = idx[:, None] >= idx[None, :]
    decay = torch.exp(diff.masked_fill(~lower_eq, 0.0)) * lower_eq       # exp(G_t - G_s) for s <= t, else 0 (never overflows)
    kk = kc @ kc.transpose(-1, -2)
    Lm = decay * kk * lower                                              # strictly lower
    sysm = torch.eye(C, device=q.device, dtype=q.dtype) + bc[..., :, None] * Lm
    eG = torch.exp(G)[..., None]
    rhs = torch.cat([bc[..., None] * vc, bc[..., None] * (eG * kc)], dim=-1)       # solve for T V and T (exp(G) K) together
    sol = torch.linalg.solve_triangular(sysm, rhs, upper=False)
    U0, W = sol[..., :dv], sol[..., dv:]                                 # U = U0 - W S0^T
    A = decay * (qc @ kc.transpose(-1, -2))                              # s <= t, diagonal included
    eQ = eG * qc
    k_end = torch.exp(G[..., -1:, None] - G[..., None]) * kc             # exp(G_end - G_s) k_s
    g_end = torch.exp(G[..., -1])[..., None, None]
    S = torch.zeros(b, h, dv, dk, dtype=q.dtype, device=q.device)
    outs = []
    for c in range(nc):                                                  # only the state crosses chunk borders
        U = U0[:, :, c] - W[:, :, c] @ S.transpose(-1, -2)               # (b, h, C, dv)
        outs.append(eQ[:, :, c] @ S.transpose(-1, -2) + A[:, :, c] @ U)
        S = g_end[:, :, c] * S + U.transpose(-1, -2) @ k_end[:, :, c]
    o = torch.stack(outs, 2).reshape(b, h, L, dv)
    return o.permute(0, 2, 1, 3)


def gated_delta_rule(q, k, v, g, beta, seg_start, chunk: int = 64):
    """Gated delta rule in chunk-parallel form (differentiable; fp32 inside):
    S <- exp(g_t) S (I - beta_t k_t k_t^T) + beta_t v_t k_t^T;  o_t = S q_t, the state reset at segment starts.
    q, k (n, h, dk) l2-normalised; v (n, h, dv); g (n, h) log-decay <= 0; beta (n, h) in (0, 1); seg_start (n,) the index of
    the first token of each token's segment.  Segments of equal length run as one batch; a ragged round runs one batch per
    length.  Same mathematics as :func:`gated_delta_rule_sequential`, which stays as its oracle; the reference calls the
    chunked kernels of the ``fla`` package here (``src/dataflow_training/model_families/qwen35/blocks.py:137-160,249-357``)."""
    n, h, dk = q.shape
    starts = torch.unique_consecutive(seg_start).tolist()               # host-known on this lane (it runs under autograd)
    bounds = starts + [n]
    lens = [bounds[i + 1] - bounds[i] for i in range(len(starts))]
    qf, kf, vf = q.float() * dk ** -0.5, k.float(), v.float()
    gf, bf = g.float(), beta.float()
    out = torch.empty(n, h, v.shape[-1], dtype=torch.float32, device=q.device)
    pieces = []
    for length in sorted(set(lens)):
        segs = [i for i, x in enumerate(lens) if x == length]
        pad = (-length) % chunk
        rows = torch.cat([torch.arange(bounds[i], bounds[i] + length, device=q.device) for i in segs])

        def take(t, fill=0.0):
            x = t[rows].reshape(len(segs), length, *t.shape[1:])
            return F.pad(x, (0, 0) * (x.dim() - 2) + (0, pad), value=fill) if pad else x
        o = _delta_rule_chunks(take(qf), take(kf), take(vf), take(gf), take(bf), chunk)
        pieces.append((rows, o[:, :length].reshape(len(segs) * length, h, -1)))
    for rows, o in pieces:
        out = out.index_copy(0, rows, o)
    return out.to(q.dtype)
