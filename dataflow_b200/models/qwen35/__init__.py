"""qwen35 family: a hybrid stack — gated delta-rule linear attention (causal depthwise convolution + SiLU on q / k / v,
l2-normalised q and k, per-head decay and write strength, gated RMSNorm on the output) in every layer except each
``full_every``-th, which is gated GQA softmax attention with per-head q / k norms and partial RoPE.  Kinds ``linattn`` and
``gattn``; the MLP is dense SwiGLU here and a mixture of experts in ``qwen35moe``.  Blocks are written in reference form
(``models/_forms.py``; the delta rule in its sequential form) and run through the autograd lane.
Family parity: reference ``src/dataflow_training/model_families/qwen35/blocks.py:83-597``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from ...blocks.layouts import DTypePolicy, Field
from .. import _forms as F
from .._torch_family import TorchFamilySpec, register_torch_family


@dataclass(frozen=True)
class Qwen35Config:
    name: str = "qwen35"
    n_layers: int = 4
    full_every: int = 4
    d_model: int = 128
    # linear-attention layers
    lin_k_heads: int = 2
    lin_v_heads: int = 4
    lin_dk: int = 16
    lin_dv: int = 16
    conv_width: int = 4
    # full-attention layers
    n_heads: int = 4
    n_kv_heads: int = 2
    head_dim: int = 32
    rope_frac: float = 0.25
    d_ff: int = 256
    # mixture of experts (qwen35moe): 0 experts = dense MLP
    n_experts: int = 0
    top_k: int = 0
    d_ff_expert: int = 0
    shared_expert: bool = False
    aux_coef: float = 0.0
    # expert parallelism (qwen35moe): this rank holds n_experts / ep routed experts
    ep: int = 1
    ep_capacity: float = 2.0
    vocab_size: int = 1024
    rope_theta: float = 10000.0
    rms_eps: float = 1e-6
    seq_len: int = 64
    batch: int = 2
    grad_accum_rounds: int = 2
    dtype_policy: Any = "bf16"
    optimizer: str = "adamw"
    optimizer_placement: str = "interleaved"
    head_chunk_tokens: int = 2048
    family: str = "qwen35"

    def policy(self) -> DTypePolicy:
        return self.dtype_policy if isinstance(self.dtype_policy, DTypePolicy) else DTypePolicy.from_dict(self.dtype_policy)

    @property
    def tokens_per_round(self) -> int:
        return self.seq_len * self.batch


def mlp_fields(c: Qwen35Config):
    d = c.d_model
    f = [Field("ffn_norm", (d,), "bf16", "vector", "ones")]
    if c.n_experts:
        f += [Field("w_router", (d, c.n_experts)), Field("w13_experts", (c.n_experts // c.ep, d, 2 * c.d_ff_expert)),
              Field("w2_experts", (c.n_experts // c.ep, c.d_ff_expert, d), "bf16", "matrix", "residual")]
        if c.shared_expert:
            f += [Field("w_shared_gate", (d, 1)), Field("w13_shared", (d, 2 * c.d_ff_expert)),
                  Field("w2_shared", (c.d_ff_expert, d), "bf16", "matrix", "residual")]
    else:
        f += [Field("w13", (d, 2 * c.d_ff)), Field("w2", (c.d_ff, d), "bf16", "matrix", "residual")]
    return f


def kind_fields(c: Qwen35Config, kind: str):
    d = c.d_model
    if kind.startswith("lin"):
        ch = 2 * c.lin_k_heads * c.lin_dk + c.lin_v_heads * c.lin_dv
        f = [Field("attn_norm", (d,), "bf16", "vector", "ones"), Field("w_qkv", (d, ch)), Field("conv_w", (ch, c.conv_width)),
             Field("w_decay", (d, c.lin_v_heads)), Field("decay_bias", (c.lin_v_heads,), "bf16", "vector", "zeros"),
             Field("a_log", (c.lin_v_heads,), "bf16", "vector", "zeros"), Field("w_beta", (d, c.lin_v_heads)),
             Field("w_gate", (d, c.lin_v_heads * c.lin_dv)), Field("o_norm", (c.lin_dv,), "bf16", "vector", "ones"),
             Field("wo", (c.lin_v_heads * c.lin_dv, d), "bf16", "matrix", "residual")]
    else:
        f = [Field("attn_norm", (d,), "bf16", "vector", "ones"), Field("w_q", (d, 2 * c.n_heads * c.head_dim)),
             Field("w_kv", (d, 2 * c.n_kv_heads * c.head_dim)), Field("q_norm", (c.head_dim,), "bf16", "vector", "ones"),
             Field("k_norm", (c.head_dim,), "bf16", "vector", "ones"), Field("wo", (c.n_heads * c.head_dim, d), "bf16", "matrix", "residual")]
    return tuple(f + mlp_fields(c))


def _seg_start(seg, n, device):
    return torch.arange(n, device=device) - seg.positions.to(device)[:n].long()


def linear_attention(c: Qwen35Config, x, w, seg):
    n = x.shape[0]
    h = F.rmsnorm(x, w["attn_norm"], c.rms_eps)
    start = _seg_start(seg, n, x.device)
    qkv = F.causal_conv1d_silu(h @ w["w_qkv"], w["conv_w"], start)
    nk = c.lin_k_heads * c.lin_dk
    q = F.l2norm(qkv[:, :nk].view(n, c.lin_k_heads, c.lin_dk))
    k = F.l2norm(qkv[:, nk:2 * nk].view(n, c.lin_k_heads, c.lin_dk))
    v = qkv[:, 2 * nk:].view(n, c.lin_v_heads, c.lin_dv)
    rep = c.lin_v_heads // c.lin_k_heads
    if rep > 1:
        q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    g = -torch.exp(w["a_log"].float()) * torch.nn.functional.softplus((h @ w["w_decay"]).float() + w["decay_bias"].float())
    beta = torch.sigmoid((h @ w["w_beta"]).float())
    o = F.gated_delta_rule(q, k, v, g, beta, start)                               # (n, hv, dv)
    gate = (h @ w["w_gate"]).view(n, c.lin_v_heads, c.lin_dv)
    o = F.gated_rmsnorm(o, gate, w["o_norm"], c.rms_eps)
    return x + o.reshape(n, -1) @ w["wo"]


def gated_attention(c: Qwen35Config, x, w, seg):
    n, hd = x.shape[0], c.head_dim
    pos = seg.positions[:n]
    h = F.rmsnorm(x, w["attn_norm"], c.rms_eps)
    qg = (h @ w["w_q"]).view(n, c.n_heads, 2 * hd)
    q, gate = qg[..., :hd], qg[..., hd:]
    kv = (h @ w["w_kv"]).view(n, c.n_kv_heads, 2 * hd)
    k, v = kv[..., :hd], kv[..., hd:]
    q, k = F.rmsnorm(q, w["q_norm"], c.rms_eps), F.rmsnorm(k, w["k_norm"], c.rms_eps)
    r = int(hd * c.rope_frac) // 2 * 2                                              # partial RoPE: the first r dims rotate
    if r:
        q = torch.cat([F.rope(q[..., :r], pos, c.rope_theta), q[..., r:]], -1)
        k = torch.cat([F.rope(k[..., :r], pos, c.rope_theta), k[..., r:]], -1)
    o, _ = F.attention(q, k, v, F.segment_causal_mask(seg, n, x.device), hd ** -0.5)
    o = o * torch.sigmoid(gate.float()).to(o.dtype)
    return x + o.reshape(n, -1) @ w["wo"]


def mlp_part(c: Qwen35Config, h_mid, w, ep=None):
    h2 = F.rmsnorm(h_mid, w["ffn_norm"], c.rms_eps)
    if not c.n_experts:
        return h_mid + F.swiglu_mlp(h2, w["w13"], w["w2"]), None
    logits = h2 @ w["w_router"]
    wts, ids = F.route_softmax_topk(logits, c.top_k)
    if ep is not None:
        y = F.moe_mlp_ep(h2, w["w13_experts"], w["w2_experts"], wts, ids, ep)
    else:
        y = F.moe_mlp(h2, w["w13_experts"], w["w2_experts"], wts, ids)
    if c.shared_expert:
        y = y + torch.sigmoid((h2 @ w["w_shared_gate"]).float()).to(y.dtype) * F.swiglu_mlp(h2, w["w13_shared"], w["w2_shared"])
    return h_mid + y, F.load_balance_aux(logits, ids, c.aux_coef)


def block_fn(c: Qwen35Config, kind: str, x, w, seg, layer, ep=None):
    h_mid = linear_attention(c, x, w, seg) if kind.startswith("lin") else gated_attention(c, x, w, seg)
    return mlp_part(c, h_mid, w, ep)


def kind_flops(c: Qwen35Config, kind: str, tokens: int):
    d = c.d_model
    mlp = d * c.n_experts + 3 * d * c.d_ff_expert * (c.top_k + (1 if c.shared_expert else 0)) if c.n_experts else 3 * d * c.d_ff
    if kind.startswith("lin"):
        ch = 2 * c.lin_k_heads * c.lin_dk + c.lin_v_heads * c.lin_dv
        p = d * ch + 2 * d * c.lin_v_heads + 2 * d * c.lin_v_heads * c.lin_dv
        return 2.0 * tokens * (p + mlp), 6.0 * tokens * c.lin_v_heads * c.lin_dk * c.lin_dv
    p = d * 2 * c.n_heads * c.head_dim + d * 2 * c.n_kv_heads * c.head_dim + c.n_heads * c.head_dim * d
    return 2.0 * tokens * (p + mlp), 2.0 * tokens * c.seq_len * c.n_heads * c.head_dim


def layer_kinds(c: Qwen35Config):
    moe = "moe" if c.n_experts else ""
    return [("gattn" if (i + 1) % c.full_every == 0 else "linattn") + moe for i in range(c.n_layers)]


PRESETS = {
    "tiny": dict(name="tiny"),
    "qwen35_9b": dict(name="qwen35_9b", n_layers=36, d_model=4096, lin_k_heads=16, lin_v_heads=32, lin_dk=128, lin_dv=128, n_heads=32,
                      n_kv_heads=8, head_dim=128, d_ff=12288, vocab_size=151936, rope_theta=1e7, seq_len=4096, batch=1, grad_accum_rounds=16,
                      dtype_policy="bf16_split_master"),
}

SPEC = TorchFamilySpec("qwen35", Qwen35Config, {k: (lambda kw=v: Qwen35Config(**kw)) for k, v in PRESETS.items()}, layer_kinds, kind_fields,
                       block_fn, kind_flops)
FAMILY = register_torch_family(SPEC)
