"""Plain PyTorch GPT-2 with autograd (LayerNorm, learned positions, GELU-tanh, optional tied head)
and the engine → ``state_dict`` bridge.  Oracle role: reference ``reference_models/gpt2.py``."""
from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F


class Gpt2Twin(nn.Module):
    def __init__(self, cfg, dtype=torch.float32):
        super().__init__()
        from ..gpt2.model import block_fields, derive_dims
        self.cfg = cfg
        self.d = d = derive_dims(cfg)
        P = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype))  # noqa: E731
        self.wte, self.wpe = P(d.vocab, d.d), P(d.n_pos, d.d)
        self.layers = nn.ModuleList()
        for _ in range(d.n_layers):
            l = nn.Module()
            for f in block_fields(d):
                setattr(l, f.name, P(*f.shape))
            self.layers.append(l)
        self.final_norm = P(d.d)
        if d.bias:
            self.final_norm_b = P(d.d)
        if not d.tied:
            self.w_head = P(d.d, d.vocab)

    def forward(self, tokens, bounds):
        d = self.d
        lens = [b - a for a, b in zip(bounds[:-1], bounds[1:])]
        pos = torch.cat([torch.arange(l, device=tokens.device) for l in lens])
        x = self.wte[tokens.long()] + self.wpe[pos]
        g = lambda l, n: getattr(l, n, None)  # noqa: E731
        for l in self.layers:
            h = F.layer_norm(x, (d.d,), l.ln1_w, g(l, "ln1_b"), d.eps)
            qkv = h @ l.c_attn_w
            if d.bias:
                qkv = qkv + l.c_attn_b
            q, k, v = (t.unflatten(1, (d.hq, d.hd)) for t in qkv.split(d.d, dim=1))
            outs = []
            for a, b in zip(bounds[:-1], bounds[1:]):
                o = F.scaled_dot_product_attention(q[a:b].transpose(0, 1)[None], k[a:b].transpose(0, 1)[None],
                                                   v[a:b].transpose(0, 1)[None], is_causal=True)[0]
                outs.append(o.transpose(0, 1).reshape(b - a, d.d))
            attn = torch.cat(outs, 0)
            h_mid = x + attn @ l.attn_proj_w + (l.attn_proj_b if d.bias else 0)
            h2 = F.layer_norm(h_mid, (d.d,), l.ln2_w, g(l, "ln2_b"), d.eps)
            fc = h2 @ l.fc_w + (l.fc_b if d.bias else 0)
            x = h_mid + F.gelu(fc, approximate="tanh") @ l.mlp_proj_w + (l.mlp_proj_b if d.bias else 0)
        xn = F.layer_norm(x, (d.d,), self.final_norm, getattr(self, "final_norm_b", None), d.eps)
        return xn @ (self.wte.t() if d.tied else self.w_head)

    def loss(self, tokens, targets, bounds, total_rows=None):
        logits = self.forward(tokens, bounds).float()
        nll = F.cross_entropy(logits, targets.long().clamp(min=0), reduction="none") * (targets >= 0).float()
        return nll.sum() / float(total_rows if total_rows is not None else max(int((targets >= 0).sum()), 1))


def state_dict_from_engine(cfg, views_of) -> dict[str, torch.Tensor]:
    from ..gpt2.model import derive_dims, family_layouts
    d = derive_dims(cfg)
    lay = family_layouts(d, cfg.policy(), cfg.optimizer)
    e = views_of("W_embed", lay.embed_w)
    sd = {"wte": e["wte"].float().clone(), "wpe": e["wpe"].float().clone()}
    for i in range(d.n_layers):
        for k, t in views_of(f"W_{i}", lay.block_w).items():
            sd[f"layers.{i}.{k}"] = t.float().clone()
    for k, t in views_of("W_head", lay.head_w).items():
        sd[k] = t.float().clone()
    return sd
