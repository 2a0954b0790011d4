"""dsv3 family (DeepSeek-V3 architecture): multi-head latent attention in every layer; the first ``n_dense`` layers
carry a dense SwiGLU MLP (kind ``mladense``), the rest a mixture of experts with sigmoid "no-aux" grouped routing and
one ungated shared expert (kind ``mlamoe``).  Blocks are written in reference form (``models/_forms.py``) and run
through the autograd lane of ``models/_torch_family.py``.
Family parity: reference ``src/dataflow_training/model_families/dsv3/{blocks.py,model.py}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from ...blocks.layouts import DTypePolicy, Field
from .. import _forms as F
from .._torch_family import TorchFamilySpec, register_torch_family


@dataclass(frozen=True)
class Dsv3Config:
    name: str = "dsv3"
    n_layers: int = 2
    n_dense: int = 1
    d_model: int = 128
    n_heads: int = 4
    q_lora: int = 48
    kv_lora: int = 32
    d_nope: int = 32
    d_rope: int = 16
    d_v: int = 32
    d_ff: int = 256
    n_experts: int = 8
    top_k: int = 2
    d_ff_expert: int = 64
    n_shared: int = 1
    n_group: int = 2
    topk_group: int = 1
    routed_scaling: float = 1.0
    vocab_size: int = 1024
    rope_theta: float = 10000.0
    rms_eps: float = 1e-6
    seq_len: int = 128
    batch: int = 2
    grad_accum_rounds: int = 2
    dtype_policy: Any = "bf16"
    optimizer: str = "adamw"
    optimizer_placement: str = "interleaved"
    head_chunk_tokens: int = 2048
    family: str = "dsv3"
    # sparse attention (dsv32): a lightning indexer picks ``index_topk`` keys per query; 0 = dense attention
    index_heads: int = 0
    index_dim: int = 0
    index_topk: int = 0
    index_kl_coef: float = 0.0
    # "mask": the selection as an (n, n) mask over dense attention (short rounds); "gather": every query attends over its
    # gathered keys in the latent form and nothing of size (n, n) exists (long context); "auto" picks by the round's length
    sparse_impl: str = "auto"
    # dense warm-up of the indexer (dsv32): attention stays DENSE, the indexer learns the full-prefix attention
    # distribution through its KL term, and nothing but the indexer's fields is updated
    dsa_warmup: bool = False
    # expert parallelism: this rank holds n_experts / ep routed experts and serves rows of every rank's tokens
    ep: int = 1
    ep_capacity: float = 2.0
    # "fp8": the dense and shared-expert MLP projections and the attention output projection run their forward on e4m3
    # operands (per-row / per-column scales); the routed experts' grouped GEMMs and every backward product stay bf16
    linear_precision: str = "bf16"

    @property
    def trainable_patterns(self) -> tuple[str, ...]:
        """fnmatch patterns of the only fields the optimizer updates (empty: all of them)."""
        return ("wi_*",) if self.dsa_warmup else ()

    def policy(self) -> DTypePolicy:
        return self.dtype_policy if isinstance(self.dtype_policy, DTypePolicy) else DTypePolicy.from_dict(self.dtype_policy)

    @property
    def tokens_per_round(self) -> int:
        return self.seq_len * self.batch


def attention_fields(c: Dsv3Config):
    d, h = c.d_model, c.n_heads
    f = [Field("attn_norm", (d,), "bf16", "vector", "ones")]
    if c.q_lora:
        f += [Field("wq_a", (d, c.q_lora)), Field("q_norm", (c.q_lora,), "bf16", "vector", "ones"),
              Field("wq_b", (c.q_lora, h * (c.d_nope + c.d_rope)))]
    else:
        f.append(Field("wq", (d, h * (c.d_nope + c.d_rope))))
    f += [Field("wkv_a", (d, c.kv_lora + c.d_rope)), Field("kv_norm", (c.kv_lora,), "bf16", "vector", "ones"),
          Field("wkv_b", (c.kv_lora, h * (c.d_nope + c.d_v))), Field("wo", (h * c.d_v, d), "bf16", "matrix", "residual")]
    if c.index_topk:
        # the indexer reads the normalised q latent (the residual stream when the query has no low-rank stack)
        f += [Field("wi_q", (c.q_lora or d, c.index_heads * c.index_dim)), Field("wi_k", (d, c.index_dim)),
              Field("wi_k_gain", (c.index_dim,), "bf16", "vector", "ones"), Field("wi_k_bias", (c.index_dim,), "bf16", "vector", "zeros"),
              Field("wi_w", (d, c.index_heads))]
    return f


def kind_fields(c: Dsv3Config, kind: str):
    d = c.d_model
    f = attention_fields(c) + [Field("ffn_norm", (d,), "bf16", "vector", "ones")]
    if kind.endswith("dense"):
        f += [Field("w13", (d, 2 * c.d_ff)), Field("w2", (c.d_ff, d), "bf16", "matrix", "residual")]
    else:
        f += [Field("w_router", (d, c.n_experts)), Field("router_bias", (c.n_experts,), "bf16", "vector", "zeros"),
              Field("w13_experts", (c.n_experts // c.ep, d, 2 * c.d_ff_expert)),
              Field("w2_experts", (c.n_experts // c.ep, c.d_ff_expert, d), "bf16", "matrix", "residual")]
        if c.n_shared:
            f += [Field("w13_shared", (d, 2 * c.n_shared * c.d_ff_expert)),
                  Field("w2_shared", (c.n_shared * c.d_ff_expert, d), "bf16", "matrix", "residual")]
    return tuple(f)


def sparse_attention_gathered(c: Dsv3Config, h, w, pos):
    """Sparse attention without anything of size (n, n): chunked index scores -> top-k rows, attention over the gathered keys
    in the latent form, and the indexer's KL objective evaluated at the selection.  Returns (o (n, heads, dv), aux)."""
    n = h.shape[0]
    q, ckv, k_rope, cq = F.mla_latents(h, w, c, pos)
    iw = {k_: w[k_] for k_ in INDEXER_FIELDS}
    sel, live = F.dsa_select(h.detach(), cq.detach(), iw, c, pos, c.index_topk)
    o, target = F.mla_sparse_attention(q, ckv, k_rope, w["wkv_b"], sel, live, c, want_target=bool(c.index_kl_coef))
    aux = None
    if c.index_kl_coef:
        aux = c.index_kl_coef * F.dsa_indexer_kl_selected(h.detach(), cq.detach(), iw, c, pos, sel, live, target) * n
    return o, aux


def attention_part(c: Dsv3Config, x, w, seg):
    """Pre-norm MLA (dense, or sparse through the indexer) + residual.  Returns (h_mid, aux)."""
    n = x.shape[0]
    pos = seg.positions[:n]
    h = F.rmsnorm(x, w["attn_norm"], c.rms_eps)
    if c.index_topk and not c.dsa_warmup and (c.sparse_impl == "gather" or (c.sparse_impl == "auto" and n > 2048)):
        o, aux = sparse_attention_gathered(c, h, w, pos)
        return x + F.linear(o.reshape(n, -1), w["wo"], c.linear_precision), aux
    q, k, v, cq = F.mla_qkv(h, w, c, pos)
    causal = F.segment_causal_mask(seg, n, x.device)
    aux, mask = None, causal
    if c.index_topk:
        scores = F.dsa_index_scores(h.detach(), cq.detach(), {k_: w[k_] for k_ in INDEXER_FIELDS}, c, pos)
        if not c.dsa_warmup:
            mask = F.dsa_topk_mask(scores.detach(), causal, c.index_topk)
    o, probs = F.attention(q, k, v, mask, (c.d_nope + c.d_rope) ** -0.5)
    if c.index_topk and c.index_kl_coef:
        aux = c.index_kl_coef * F.dsa_indexer_kl(scores, probs, mask) * n
    return x + F.linear(o.reshape(n, -1), w["wo"], c.linear_precision), aux


EP_FIELDS = ("w13_experts", "w2_experts")
INDEXER_FIELDS = ("wi_q", "wi_k", "wi_k_gain", "wi_k_bias", "wi_w")


def routed_experts(h2, w, wts, ids, ep=None):
    """The routed experts' output: all experts here, or (``ep``: an expert-parallel group) this rank's share of them with
    the rows exchanged through the group."""
    if ep is not None:
        return F.moe_mlp_ep(h2, w["w13_experts"], w["w2_experts"], wts, ids, ep)
    return F.moe_mlp(h2, w["w13_experts"], w["w2_experts"], wts, ids)


def block_fn(c: Dsv3Config, kind: str, x, w, seg, layer, ep=None):
    h_mid, aux = attention_part(c, x, w, seg)
    h2 = F.rmsnorm(h_mid, w["ffn_norm"], c.rms_eps)
    if kind.endswith("dense"):
        return h_mid + F.swiglu_mlp(h2, w["w13"], w["w2"], c.linear_precision), aux
    logits = h2 @ w["w_router"]
    wts, ids = F.route_sigmoid_noaux(logits, w["router_bias"].detach(), c.top_k, c.n_group, c.topk_group, c.routed_scaling)
    y = routed_experts(h2, w, wts, ids, ep)
    if c.n_shared:
        y = y + F.swiglu_mlp(h2, w["w13_shared"], w["w2_shared"], c.linear_precision)
    return h_mid + y, aux


def kind_flops(c: Dsv3Config, kind: str, tokens: int):
    d, h = c.d_model, c.n_heads
    attn_p = (d * c.q_lora + c.q_lora * h * (c.d_nope + c.d_rope) if c.q_lora else d * h * (c.d_nope + c.d_rope)) + \
        d * (c.kv_lora + c.d_rope) + c.kv_lora * h * (c.d_nope + c.d_v) + h * c.d_v * d
    if c.index_topk:
        attn_p += (c.q_lora or d) * c.index_heads * c.index_dim + d * (c.index_dim + c.index_heads)
    mlp_p = 3 * d * c.d_ff if kind.endswith("dense") else d * c.n_experts + 3 * d * c.d_ff_expert * (c.top_k + c.n_shared)
    keys = min(c.index_topk, c.seq_len) if c.index_topk else c.seq_len / 2
    attn = 2.0 * tokens * keys * h * (c.d_nope + c.d_rope + c.d_v)
    if c.index_topk:
        attn += 2.0 * tokens * c.seq_len / 2 * c.index_heads * c.index_dim
    return 2.0 * tokens * (attn_p + mlp_p), attn


def layer_kinds(c: Dsv3Config):
    return ["mladense" if i < c.n_dense else "mlamoe" for i in range(c.n_layers)]


PRESETS = {
    "tiny": dict(name="tiny"),
    "dsv3_mini": dict(name="dsv3_mini", n_layers=6, n_dense=1, d_model=512, n_heads=8, q_lora=192, kv_lora=128, d_nope=64, d_rope=32, d_v=64,
                      d_ff=1408, n_experts=16, top_k=4, d_ff_expert=256, n_group=4, topk_group=2, vocab_size=32000, seq_len=1024, batch=4,
                      grad_accum_rounds=4),
    "dsv3_671b": dict(name="dsv3_671b", n_layers=61, n_dense=3, d_model=7168, n_heads=128, q_lora=1536, kv_lora=512, d_nope=128, d_rope=64,
                      d_v=128, d_ff=18432, n_experts=256, top_k=8, d_ff_expert=2048, n_group=8, topk_group=4, routed_scaling=2.5,
                      vocab_size=129280, seq_len=4096, batch=1, grad_accum_rounds=16, dtype_policy="bf16_split_master"),
}

SPEC = TorchFamilySpec("dsv3", Dsv3Config, {k: (lambda kw=v: Dsv3Config(**kw)) for k, v in PRESETS.items()}, layer_kinds, kind_fields,
                       block_fn, kind_flops, ep_fields=EP_FIELDS)
FAMILY = register_torch_family(SPEC)
