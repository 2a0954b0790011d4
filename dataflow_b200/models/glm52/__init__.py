"""glm52 family: the dsv32 architecture (multi-head latent attention, sparse attention through a lightning indexer,
mixture of experts after the first dense layers) with CROSS-LAYER INDEX SHARING: layers come in groups of
``index_share``; the first layer of a group (the leader) runs the indexer and stores the keys it selected in its context
object, the others (followers) carry no indexer weights and attend over the leader's selection.  Kinds ``gdl`` / ``gdf``
(dense leader / follower) and ``gml`` / ``gmf`` (mixture-of-experts leader / follower).  A lowering post-pass makes the
followers' forward and backward tasks read the leader's context object.
The indexer is trained against the attention of EVERY layer that uses its selection: each follower's backward adds its
target (head-summed attention probabilities, L1-normalised per query, gathered at the shared selection) to the group's
accumulator object, and the leader's backward — the last of the group to run — takes the KL of its index distribution
to ``(own target + the followers' sum) / group size``.  A leader without followers keeps dsv32's per-layer rule.
Reference role: ``src/dataflow_training/model_families/glm52/{blocks.py,model.py}``.
"""
from __future__ import annotations

import dataclasses

import torch

from ...blocks.layouts import Field
from .. import _forms as F
from ..dsv3 import EP_FIELDS, INDEXER_FIELDS, Dsv3Config, kind_fields as _dsv3_fields, kind_flops as _dsv3_flops, routed_experts
from .._torch_family import TorchFamilySpec, register_torch_family


@dataclasses.dataclass(frozen=True)
class Glm52Config(Dsv3Config):
    index_share: int = 2
    # One role per layer, "full" (runs the indexer) or "shared" (attends over the nearest earlier full layer's selection);
    # empty = regular groups of ``index_share`` layers.  Published checkpoints carry a searched, irregular pattern.
    indexer_types: tuple = ()

    def __post_init__(self):
        parent = getattr(super(), "__post_init__", None)
        if parent is not None:
            parent()
        t = tuple(self.indexer_types)
        if t:
            if len(t) != self.n_layers or t[0] != "full" or any(r not in ("full", "shared") for r in t):
                raise ValueError("indexer_types needs one of full|shared per layer, and layer 0 must be full")
            object.__setattr__(self, "indexer_types", t)


def roles(c: Glm52Config):
    """Per layer ``"full"`` or ``"shared"``."""
    if c.indexer_types:
        return tuple(c.indexer_types)
    return tuple("full" if i % c.index_share == 0 else "shared" for i in range(c.n_layers))


def leader_of(c: Glm52Config, layer: int):
    r = roles(c)
    if r[layer] == "full":
        return None
    lead = layer
    while r[lead] != "full":
        lead -= 1
    return lead


def layer_kinds(c: Glm52Config):
    return [("gd" if i < c.n_dense else "gm") + ("l" if leader_of(c, i) is None else "f") for i in range(c.n_layers)]


def kind_fields(c: Glm52Config, kind: str):
    f = _dsv3_fields(c, "x_dense" if kind.startswith("gd") else "x_moe")
    return tuple(x for x in f if kind.endswith("l") or not x.name.startswith("wi_"))


def ctx_fields(c: Glm52Config, tokens: int):
    return (Field("sel", (tokens, min(c.index_topk, c.seq_len)), "int32"),)


def accum_fields(c: Glm52Config, tokens: int):
    return (Field("kl_target", (tokens, min(c.index_topk, c.seq_len)), "fp32"),)


def block_fn(c: Glm52Config, kind: str, x, w, seg, layer, shared=None, accum=None, group_size=1, ep=None):
    n = x.shape[0]
    pos = seg.positions[:n]
    h = F.rmsnorm(x, w["attn_norm"], c.rms_eps)
    aux, emit = None, None
    width = min(c.index_topk, c.seq_len)
    if c.sparse_impl == "gather" or (c.sparse_impl == "auto" and n > 2048):
        # long context: nothing of size (n, n); dead slots of the published selection hold -1
        q, ckv, k_rope, cq = F.mla_latents(h, w, c, pos)
        pad = torch.nn.functional.pad
        if shared is None:
            iw = {k_: w[k_] for k_ in INDEXER_FIELDS}
            sel, live = F.dsa_select(h.detach(), cq.detach(), iw, c, pos, width)
            emit = {"sel": pad(torch.where(live, sel, torch.full_like(sel, -1)), (0, width - sel.shape[1]), value=-1).to(torch.int32)}
        else:
            got = shared["sel"].long()[:, :min(width, n)]
            sel, live = got.clamp(min=0), got >= 0
        o, target = F.mla_sparse_attention(q, ckv, k_rope, w["wkv_b"], sel, live, c, want_target=bool(c.index_kl_coef))
        if c.index_kl_coef:
            if shared is not None:
                emit = {"_deposit": {"kl_target": pad(target, (0, width - target.shape[1]))}}
            else:
                if accum is not None:
                    target = (target + accum["kl_target"][:, :target.shape[1]].to(target.dtype)) / group_size
                aux = c.index_kl_coef * F.dsa_indexer_kl_selected(h.detach(), cq.detach(), iw, c, pos, sel, live, target) * n
    else:
        q, k, v, cq = F.mla_qkv(h, w, c, pos)
        causal = F.segment_causal_mask(seg, n, x.device)
        if shared is None:                                              # leader: rank the keys, publish the selection
            scores = F.dsa_index_scores(h.detach(), cq.detach(), {k_: w[k_] for k_ in INDEXER_FIELDS}, c, pos)
            kk = min(c.index_topk, c.seq_len, n)
            sel = scores.detach().masked_fill(~causal, float("-inf")).topk(kk, dim=-1).indices
            emit = {"sel": torch.nn.functional.pad(sel, (0, min(c.index_topk, c.seq_len) - kk)).to(torch.int32)}
        else:
            sel = shared["sel"].long()[:, :min(c.index_topk, c.seq_len, n)]
        mask = torch.zeros_like(causal).scatter_(1, sel.clamp(max=n - 1), True) & causal
        o, probs = F.attention(q, k, v, mask, (c.d_nope + c.d_rope) ** -0.5)
        if c.index_kl_coef:
            target = F.dsa_attention_target(probs)
            cols = sel.clamp(max=n - 1)
            if shared is not None:                                      # follower: its share of the leader's target
                width = min(c.index_topk, c.seq_len)
                emit = {"_deposit": {"kl_target": torch.nn.functional.pad(target.gather(1, cols), (0, width - cols.shape[1]))}}
            else:
                if accum is not None:
                    target = (target + torch.zeros_like(target).scatter_add_(1, cols, accum["kl_target"][:, :cols.shape[1]].to(target.dtype))) / group_size
                aux = c.index_kl_coef * F.dsa_indexer_kl_to(scores, target, mask) * n
    h_mid = x + F.linear(o.reshape(n, -1), w["wo"], c.linear_precision)
    h2 = F.rmsnorm(h_mid, w["ffn_norm"], c.rms_eps)
    if kind.startswith("gd"):
        y = F.swiglu_mlp(h2, w["w13"], w["w2"], c.linear_precision)
    else:
        wts, ids = F.route_sigmoid_noaux(h2 @ w["w_router"], w["router_bias"].detach(), c.top_k, c.n_group, c.topk_group, c.routed_scaling)
        y = routed_experts(h2, w, wts, ids, ep)
        if c.n_shared:
            y = y + F.swiglu_mlp(h2, w["w13_shared"], w["w2_shared"], c.linear_precision)
    return h_mid + y, aux, emit


def kind_flops(c: Glm52Config, kind: str, tokens: int):
    mm, at = _dsv3_flops(c, "x_dense" if kind.startswith("gd") else "x_moe", tokens)
    if kind.endswith("f"):                                          # followers run no indexer
        mm -= 2.0 * tokens * ((c.q_lora or c.d_model) * c.index_heads * c.index_dim + c.d_model * (c.index_dim + c.index_heads))
        at -= 2.0 * tokens * c.seq_len / 2 * c.index_heads * c.index_dim
    return mm, at


def pattern(*runs):
    """("full", 3), ("shared", 3), (("full", "shared", "shared", "shared"), 18) -> the flat tuple of roles."""
    out = []
    for what, times in runs:
        out += (list(what) if isinstance(what, tuple) else [what]) * times
    return tuple(out)


BASE = dict(index_heads=2, index_dim=16, index_topk=32, index_kl_coef=0.1, index_share=2, family="glm52")
PRESETS = {
    "tiny": dict(name="tiny", n_layers=4, n_dense=2, **BASE),
    "glm52_mini": dict(name="glm52_mini", n_layers=8, n_dense=2, d_model=512, n_heads=8, q_lora=192, kv_lora=128, d_nope=64, d_rope=32, d_v=64,
                       d_ff=1408, n_experts=16, top_k=4, d_ff_expert=256, n_group=4, topk_group=2, vocab_size=32000, seq_len=1024, batch=4,
                       grad_accum_rounds=4, **{**BASE, "index_heads": 4, "index_dim": 32, "index_topk": 256, "index_share": 4}),
    # the published model: wide heads (192 + 64 query/key dims, 256 value dims), one routing group, and a searched sharing
    # pattern — three full layers, three shared, then eighteen groups of one full and three shared
    "glm52": dict(name="glm52", n_layers=78, n_dense=3, d_model=6144, n_heads=64, q_lora=2048, kv_lora=512, d_nope=192, d_rope=64, d_v=256,
                  d_ff=12288, n_experts=256, top_k=8, d_ff_expert=2048, n_group=1, topk_group=1, routed_scaling=2.5, vocab_size=154880,
                  seq_len=4096, batch=1, grad_accum_rounds=16, dtype_policy="bf16_split_master",
                  indexer_types=pattern(("full", 3), ("shared", 3), (("full", "shared", "shared", "shared"), 18)),
                  **{**BASE, "index_heads": 32, "index_dim": 128, "index_topk": 2048, "index_share": 4}),
}

SPEC = TorchFamilySpec("glm52", Glm52Config, {k: (lambda kw=v: Glm52Config(**kw)) for k, v in PRESETS.items()}, layer_kinds, kind_fields,
                       block_fn, kind_flops, ctx_fields=ctx_fields, leader_of=leader_of, accum_fields=accum_fields, ep_fields=EP_FIELDS)
FAMILY = register_torch_family(SPEC)
