"""Plain PyTorch Llama-3 (RMSNorm, GQA, rotate-half RoPE, SwiGLU) with autograd, plus the
bridge that maps engine bytes to its ``state_dict``.  Weights keep the engine's
``(in, out)`` orientation and fused packing so the bridge is a copy, not a transpose.
Oracle role: reference ``reference_models/llama3.py`` + ``model_families/llama3/bridge.py``.
"""
from __future__ import annotations

import math

import torch
from torch import nn


def _rope(x, positions, theta):
    # x: (t, h, d)
    d = x.shape[-1]
    half = d // 2
    inv = torch.exp2(-math.log2(theta) * (2.0 * torch.arange(half, device=x.device, dtype=torch.float32) / d))
    ang = positions.float().unsqueeze(-1) * inv
    cs, sn = torch.cos(ang).unsqueeze(1), torch.sin(ang).unsqueeze(1)
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([a * cs - b * sn, b * cs + a * sn], -1).to(x.dtype)


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


class Llama3Twin(nn.Module):
    def __init__(self, cfg, dtype=torch.float32):
        super().__init__()
        from ..llama3.model import derive_dims
        self.cfg = cfg
        self.d = d = derive_dims(cfg)
        P = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype))  # noqa: E731
        self.wte = P(d.vocab, d.d)
        self.layers = nn.ModuleList()
        for _ in range(d.n_layers):
            l = nn.Module()
            l.attn_norm, l.w_qkv, l.wo = P(d.d), P(d.d, d.qkv_dim), P(d.q_dim, d.d)
            l.ffn_norm = P(d.d)
            if d.moe:
                l.w_router, l.w13_experts, l.w2_experts = P(d.d, d.E), P(d.E, d.d, 2 * d.Fe), P(d.E, d.Fe, d.d)
            else:
                l.w13, l.w2 = P(d.d, 2 * d.F), P(d.F, d.d)
            if d.qk_norm:
                l.q_norm, l.k_norm = (P(d.q_dim), P(d.kv_dim)) if d.qk_norm == "full" else (P(d.hd), P(d.hd))
            self.layers.append(l)
        self.final_norm, self.w_head = P(d.d), P(d.d, d.vocab)

    def forward(self, tokens, bounds):
        """tokens (t,) int; bounds: sequence boundaries [0, b1, ..., t].  Returns logits (t, vocab)."""
        d = self.d
        lens = [b - a for a, b in zip(bounds[:-1], bounds[1:])]
        pos = torch.cat([torch.arange(l, device=tokens.device) for l in lens])
        x = self.wte[tokens.long()]
        for l in self.layers:
            h = _rms(x, l.attn_norm, d.eps)
            qkv = h @ l.w_qkv
            q = qkv[:, :d.q_dim].unflatten(1, (d.hq, d.hd))
            k = qkv[:, d.q_dim:d.q_dim + d.kv_dim].unflatten(1, (d.hkv, d.hd))
            v = qkv[:, d.q_dim + d.kv_dim:].unflatten(1, (d.hkv, d.hd))
            if d.qk_norm == "full":
                q, k = _rms(q.flatten(1), l.q_norm, d.eps).view_as(q), _rms(k.flatten(1), l.k_norm, d.eps).view_as(k)
            elif d.qk_norm:
                q, k = _rms(q, l.q_norm, d.eps), _rms(k, l.k_norm, d.eps)
            q, k = _rope(q, pos, d.theta), _rope(k, pos, d.theta)
            outs = []
            rep = d.hq // d.hkv
            for a, b in zip(bounds[:-1], bounds[1:]):
                qs = q[a:b].transpose(0, 1)
                ks = k[a:b].transpose(0, 1).repeat_interleave(rep, 0)
                vs = v[a:b].transpose(0, 1).repeat_interleave(rep, 0)
                o = torch.nn.functional.scaled_dot_product_attention(qs[None], ks[None], vs[None], is_causal=True)[0]
                outs.append(o.transpose(0, 1).reshape(b - a, d.q_dim))
            attn = torch.cat(outs, 0)
            h_mid = x + attn @ l.wo
            h2 = _rms(h_mid, l.ffn_norm, d.eps)
            if d.moe:
                x = h_mid + self._moe(l, h2)
            else:
                h13 = h2 @ l.w13
                s = torch.nn.functional.silu(h13[:, :d.F]) * h13[:, d.F:]
                x = h_mid + s @ l.w2
        return _rms(x, self.final_norm, d.eps) @ self.w_head

    def _moe(self, l, h2):
        """Dense-loop mixture of experts: the same selection rule as the engine (ties to the smallest index),
        differentiable route weights."""
        from ...ops.eager import moe_topk_softmax
        d = self.d
        logits = h2 @ l.w_router
        _, ids = moe_topk_softmax(logits.detach(), d.topk, d.routing_mode)
        ids = ids.long()
        if d.routing_mode == "topk_then_softmax":
            w = torch.softmax(logits.float().gather(1, ids), -1)
        else:
            w = torch.softmax(logits.float(), -1).gather(1, ids)
        out = torch.zeros_like(h2)
        for e in range(d.E):
            tok, slot = (ids == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            h13 = h2[tok] @ l.w13_experts[e]
            s = torch.nn.functional.silu(h13[:, :d.Fe]) * h13[:, d.Fe:]
            out = out.index_add(0, tok, (s @ l.w2_experts[e]) * w[tok, slot].unsqueeze(-1).to(h2.dtype))
        return out

    def loss(self, tokens, targets, bounds, total_rows=None):
        logits = self.forward(tokens, bounds).float()
        nll = torch.nn.functional.cross_entropy(logits, targets.long().clamp(min=0), reduction="none")
        nll = nll * (targets >= 0).float()
        return nll.sum() / float(total_rows if total_rows is not None else max(int((targets >= 0).sum()), 1))


def state_dict_from_engine(cfg, views_of) -> dict[str, torch.Tensor]:
    """Engine store bytes → twin ``state_dict`` (fp32 copies)."""
    from ..llama3.model import derive_dims, family_layouts
    d = derive_dims(cfg)
    lay = family_layouts(d, cfg.policy(), cfg.optimizer)
    sd = {"wte": views_of("W_embed", lay.embed_w)["wte"].float().clone()}
    for i in range(d.n_layers):
        w = views_of(f"W_{i}", lay.block_w)
        for k, t in w.items():
            sd[f"layers.{i}.{k}"] = t.float().clone()
    h = views_of("W_head", lay.head_w)
    sd["final_norm"], sd["w_head"] = h["final_norm"].float().clone(), h["w_head"].float().clone()
    return sd
