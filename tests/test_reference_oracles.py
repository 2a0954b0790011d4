"""Independent oracles: this repository's twins (and through them the engine, which the family gates tie to the twins)
against the self-contained ``nn.Module`` per family that the reference keeps as its truth tree (``reference_models/``).
The two trees share no code: a wrong formula on one side shows up as a different loss or gradient.

The reference package is an optional, separately installed oracle (``baseline/_ref``); without it these tests skip.
Weights are generated here and carried into the reference module through an explicit map ``reference parameter <- linear
function of this repository's parameters`` (``nn.Linear`` stores (out, in), the packed fields here (in, out); some fields
are packed differently).  Both models run the same tokens in fp32; the losses must agree, and so must every gradient —
the same linear function applied to this repository's gradients gives the reference's.
"""
import dataclasses
import os
import sys

import pytest
import torch

REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "reference_models")),
                                reason="the reference's truth tree is not installed under baseline/_ref")


def ref_module(name):
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import importlib
    return importlib.import_module(f"reference_models.{name}")


def fill(module, seed):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for k, p in module.state_dict().items():
            if not p.dtype.is_floating_point:
                continue
            if p.dim() == 1:
                p.copy_(0.1 * torch.randn(p.shape, generator=g) + (0.0 if "bias" in k or "a_log" in k else 1.0))
            else:
                p.copy_(torch.randn(p.shape, generator=g) * p.shape[-2] ** -0.5)


def check(mine, theirs, pairs, my_loss, their_loss, loss_rtol=2e-4, grad_tol=5e-3):
    """``pairs``: reference parameter name -> function of a dict of this repository's tensors (parameters, then gradients)."""
    sd_t = theirs.state_dict()
    params = {k: v.detach() for k, v in mine.state_dict().items()}
    with torch.no_grad():
        for name, fn in pairs.items():
            sd_t[name].copy_(fn(params))
    left = [k for k, v in theirs.named_parameters() if k not in pairs]
    assert not left, f"reference parameters without a counterpart: {left}"
    lm, lt = my_loss(mine), their_loss(theirs)
    lt, objective = lt if isinstance(lt, tuple) else (lt, lt)     # (reported loss, what is differentiated) when they differ
    assert lm.item() == pytest.approx(lt.item(), rel=loss_rtol), (lm.item(), lt.item())
    lm.backward()
    objective.backward()
    grads = {k: (p.grad if p.grad is not None else torch.zeros_like(p)) for k, p in mine.named_parameters()}
    for k, v in mine.state_dict().items():
        grads.setdefault(k, torch.zeros_like(v))
    pt = dict(theirs.named_parameters())
    for name, fn in pairs.items():
        if name not in pt or pt[name].grad is None:        # a buffer there, or a parameter the loss does not reach
            continue
        want, got = pt[name].grad, fn(grads)
        err = float((got - want).norm() / (want.norm() + 1e-12))
        assert err < grad_tol, (name, err)
    return lm.item()


def T(key):
    return lambda S: S[key].t()


def I(key):
    return lambda S: S[key]


def cols(key, lo, hi):
    return lambda S: S[key][:, lo:hi].t()


def data(vocab, B, L, seed=2):
    g = torch.Generator().manual_seed(seed)
    tokens = torch.randint(0, vocab, (B * L,), generator=g)
    targets = torch.randint(0, vocab, (B * L,), generator=g)
    return tokens, targets, [i * L for i in range(B + 1)]


def mla_pairs(i, pre="attn."):
    return {f"blocks.{i}.attn_norm.weight": I(f"layers.{i}.attn_norm"),
            f"blocks.{i}.{pre}w_q_a.weight": T(f"layers.{i}.wq_a"), f"blocks.{i}.{pre}q_a_norm.weight": I(f"layers.{i}.q_norm"),
            f"blocks.{i}.{pre}w_q_b.weight": T(f"layers.{i}.wq_b"), f"blocks.{i}.{pre}w_kv_a.weight": T(f"layers.{i}.wkv_a"),
            f"blocks.{i}.{pre}kv_a_norm.weight": I(f"layers.{i}.kv_norm"), f"blocks.{i}.{pre}w_kv_b.weight": T(f"layers.{i}.wkv_b"),
            f"blocks.{i}.{pre}wo.weight": T(f"layers.{i}.wo"), f"blocks.{i}.ffn_norm.weight": I(f"layers.{i}.ffn_norm")}


def test_dsv3_twin_matches_the_reference_truth_tree():
    """Multi-head latent attention (two low-rank stacks, decoupled rope key shared by the heads, nope-first layout), the dense
    SwiGLU layer, and the sigmoid no-aux grouped router with an ungated shared expert."""
    from dataflow_b200.models.families import resolve_family
    R = ref_module("dsv3")
    fam = resolve_family("dsv3")
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32", rms_eps=1e-5)
    mine = fam.twin(cfg)
    fill(mine, 1)
    with torch.no_grad():
        for k, p in mine.state_dict().items():
            if k.endswith("router_bias"):
                p.zero_()
    theirs = R.Dsv3(R.Dsv3Config(
        n_layers=cfg.n_layers, d_model=cfg.d_model, n_heads=cfg.n_heads, q_lora_rank=cfg.q_lora, kv_lora_rank=cfg.kv_lora,
        qk_nope_dim=cfg.d_nope, qk_rope_dim=cfg.d_rope, v_head_dim=cfg.d_v, first_k_dense=cfg.n_dense, d_ff_dense=cfg.d_ff,
        n_experts=cfg.n_experts, top_k=cfg.top_k, d_ff_expert=cfg.d_ff_expert, n_group=cfg.n_group, topk_group=cfg.topk_group,
        n_shared_experts=cfg.n_shared, d_ff_shared=cfg.n_shared * cfg.d_ff_expert, vocab_size=cfg.vocab_size,
        routed_scaling=cfg.routed_scaling, rope_base=cfg.rope_theta))
    pairs = {"embed.weight": I("wte"), "final_norm.weight": I("final_norm"), "lm_head.weight": T("w_head")}
    F_ = cfg.d_ff
    for i in range(cfg.n_layers):
        pairs.update(mla_pairs(i))
        if i < cfg.n_dense:      # [gate | up] packed into one (d, 2F) field here, two Linear layers there
            pairs.update({f"blocks.{i}.ffn.w1.weight": cols(f"layers.{i}.w13", 0, F_), f"blocks.{i}.ffn.w3.weight": cols(f"layers.{i}.w13", F_, 2 * F_),
                          f"blocks.{i}.ffn.w2.weight": T(f"layers.{i}.w2")})
        else:
            pairs.update({f"blocks.{i}.ffn.router.weight": T(f"layers.{i}.w_router"), f"blocks.{i}.ffn.w13": I(f"layers.{i}.w13_experts"),
                          f"blocks.{i}.ffn.w2": I(f"layers.{i}.w2_experts"), f"blocks.{i}.ffn.w_s13.weight": T(f"layers.{i}.w13_shared"),
                          f"blocks.{i}.ffn.w_s2.weight": T(f"layers.{i}.w2_shared")})
    B, L = 2, 48
    tokens, targets, bounds = data(cfg.vocab_size, B, L)
    check(mine, theirs, pairs, lambda m: m.loss(tokens, targets, bounds, total_rows=B * L),
          lambda m: m.loss(tokens.view(B, L), targets.view(B, L)))


def qwen35_pairs(cfg, i, kind):
    d, hd, H, KV = cfg.d_model, cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
    p = {f"blocks.{i}.attn_norm.weight": I(f"layers.{i}.attn_norm"), f"blocks.{i}.ffn_norm.weight": I(f"layers.{i}.ffn_norm")}
    L = f"layers.{i}."
    if kind == "lin":
        p.update({
            # [q | k | v] through the convolution, then the output gate z
            f"blocks.{i}.mixer.w_qkvz.weight": lambda S: torch.cat([S[L + "w_qkv"], S[L + "w_gate"]], 1).t(),
            # [beta | decay] pre-activations
            f"blocks.{i}.mixer.w_ba.weight": lambda S: torch.cat([S[L + "w_beta"], S[L + "w_decay"]], 1).t(),
            f"blocks.{i}.mixer.conv.weight": lambda S: S[L + "conv_w"].unsqueeze(1),
            f"blocks.{i}.mixer.A_log": I(L + "a_log"), f"blocks.{i}.mixer.dt_bias": I(L + "decay_bias"),
            f"blocks.{i}.mixer.lin_norm.weight": I(L + "o_norm"), f"blocks.{i}.mixer.w_out.weight": T(L + "wo")})
    else:
        # here every head keeps [q | gate] (and [k | v]) side by side; there all q precede all gates
        p.update({
            f"blocks.{i}.mixer.wq.weight": lambda S: torch.cat([S[L + "w_q"].view(d, H, 2, hd)[:, :, 0].reshape(d, H * hd),
                                                                 S[L + "w_q"].view(d, H, 2, hd)[:, :, 1].reshape(d, H * hd)], 1).t(),
            f"blocks.{i}.mixer.wk.weight": lambda S: S[L + "w_kv"].view(d, KV, 2, hd)[:, :, 0].reshape(d, KV * hd).t(),
            f"blocks.{i}.mixer.wv.weight": lambda S: S[L + "w_kv"].view(d, KV, 2, hd)[:, :, 1].reshape(d, KV * hd).t(),
            f"blocks.{i}.mixer.q_norm.weight": I(L + "q_norm"), f"blocks.{i}.mixer.k_norm.weight": I(L + "k_norm"),
            f"blocks.{i}.mixer.wo.weight": T(L + "wo")})
    return p


def test_qwen35_twin_matches_the_reference_truth_tree():
    """Gated DeltaNet (causal convolution + SiLU, l2-normalised q / k, the gated delta rule in its chunk-parallel form here
    against the reference's token-by-token recurrence, gated RMSNorm) in three of four layers, gated attention with per-head
    qk-norm and partial RoPE in the fourth; uniform and packed (ragged) rounds."""
    from dataflow_b200.models.families import resolve_family
    R = ref_module("qwen35")
    fam = resolve_family("qwen35")
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32", rms_eps=1e-5)
    mine = fam.twin(cfg)
    fill(mine, 4)
    rc = R.Qwen35Config(n_layers=cfg.n_layers, d_model=cfg.d_model, full_attention_interval=cfg.full_every, n_heads=cfg.n_heads,
                        n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, partial_rotary_factor=cfg.rope_frac, lin_k_heads=cfg.lin_k_heads,
                        lin_v_heads=cfg.lin_v_heads, lin_k_head_dim=cfg.lin_dk, lin_v_head_dim=cfg.lin_dv, lin_conv_kernel=cfg.conv_width,
                        d_ff=cfg.d_ff, vocab_size=cfg.vocab_size, rope_base=cfg.rope_theta)
    F_ = cfg.d_ff
    for shape in ("uniform", "ragged"):
        theirs = R.Qwen35(rc)
        pairs = {"embed.weight": I("wte"), "final_norm.weight": I("final_norm"), "lm_head.weight": T("w_head")}
        for i in range(cfg.n_layers):
            pairs.update(qwen35_pairs(cfg, i, rc.kind_of(i)))
            pairs.update({f"blocks.{i}.mlp.w1.weight": cols(f"layers.{i}.w13", 0, F_), f"blocks.{i}.mlp.w3.weight": cols(f"layers.{i}.w13", F_, 2 * F_),
                          f"blocks.{i}.mlp.w2.weight": T(f"layers.{i}.w2")})
        for p in mine.parameters():
            p.grad = None
        if shape == "uniform":
            B, L = 2, 40
            tokens, targets, bounds = data(cfg.vocab_size, B, L, seed=5)
            theirs_loss = lambda m: m.loss(tokens.view(B, L), targets.view(B, L))       # noqa: E731
        else:
            lens = (23, 9, 48)
            tokens, targets, _ = data(cfg.vocab_size, 1, sum(lens), seed=6)
            bounds = [0, 23, 32, 80]
            theirs_loss = lambda m: m.loss(tokens.view(1, -1), targets.view(1, -1), seq_lens=lens)       # noqa: E731
        check(mine, theirs, pairs, lambda m: m.loss(tokens, targets, bounds, total_rows=tokens.numel()), theirs_loss)


def test_qwen35moe_twin_matches_the_reference_truth_tree():
    """The hybrid stack with a mixture of experts in every layer: top-k-then-softmax routing (smallest-index tie-break), packed
    [x1 | x3] expert stacks, one sigmoid-gated shared expert; cross-entropy only (the balance term is a separate objective)."""
    from dataflow_b200.models.families import resolve_family
    R = ref_module("qwen35moe")
    fam = resolve_family("qwen35moe")
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32", rms_eps=1e-5, aux_coef=0.0)
    mine = fam.twin(cfg)
    fill(mine, 7)
    rc = R.Qwen35MoeConfig(n_layers=cfg.n_layers, d_model=cfg.d_model, full_attention_interval=cfg.full_every, n_heads=cfg.n_heads,
                           n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, partial_rotary_factor=cfg.rope_frac,
                           lin_k_heads=cfg.lin_k_heads, lin_v_heads=cfg.lin_v_heads, lin_k_head_dim=cfg.lin_dk, lin_v_head_dim=cfg.lin_dv,
                           lin_conv_kernel=cfg.conv_width, n_experts=cfg.n_experts, top_k=cfg.top_k, d_ff_expert=cfg.d_ff_expert,
                           n_shared_experts=1, d_ff_shared=cfg.d_ff_expert, vocab_size=cfg.vocab_size, rope_base=cfg.rope_theta)
    theirs = R.Qwen35Moe(rc)
    pairs = {"embed.weight": I("wte"), "final_norm.weight": I("final_norm"), "lm_head.weight": T("w_head")}
    for i in range(cfg.n_layers):
        pairs.update(qwen35_pairs(cfg, i, rc.kind_of(i)))
        pairs.update({f"blocks.{i}.moe.router.weight": T(f"layers.{i}.w_router"), f"blocks.{i}.moe.w13": I(f"layers.{i}.w13_experts"),
                      f"blocks.{i}.moe.w2": I(f"layers.{i}.w2_experts"), f"blocks.{i}.moe.shared_gate.weight": T(f"layers.{i}.w_shared_gate"),
                      f"blocks.{i}.moe.shared_up.weight": T(f"layers.{i}.w13_shared"), f"blocks.{i}.moe.shared_down.weight": T(f"layers.{i}.w2_shared")})
    B, L = 2, 40
    tokens, targets, bounds = data(cfg.vocab_size, B, L, seed=8)
    check(mine, theirs, pairs, lambda m: m.loss(tokens, targets, bounds, total_rows=B * L),
          lambda m: m.loss(tokens.view(B, L), targets.view(B, L)))


def dsa_pairs(i):
    L = f"layers.{i}."
    p = mla_pairs(i)
    p.update({f"blocks.{i}.attn.w_idx_q.weight": T(L + "wi_q"), f"blocks.{i}.attn.w_idx_k.weight": T(L + "wi_k"),
              f"blocks.{i}.attn.idx_k_ln_w": I(L + "wi_k_gain"), f"blocks.{i}.attn.idx_k_ln_b": I(L + "wi_k_bias"),
              f"blocks.{i}.attn.w_idx_w": I(L + "wi_w")})
    return p


def test_dsv32_twin_matches_the_reference_truth_tree():
    """DeepSeek sparse attention: the lightning indexer (queries from the normalised q latent, LayerNorm'd shared key, rotation
    of the first rope dims only, ReLU scores weighted per head), top-k selection, attention over the selection — and the
    indexer's KL objective over the selection's live set, whose gradient reaches the indexer's fields only."""
    from dataflow_b200.models.families import resolve_family
    R = ref_module("dsv32")
    fam = resolve_family("dsv32")
    base = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32", rms_eps=1e-5)
    # ReLU leaves many index scores at exactly zero, and the order of tied keys in a top-k is the library's business: a
    # sparse case therefore runs as ONE sequence (identical score rows on both sides, hence identical selections), and the
    # two-sequence case selects every visible key.
    for B, L, topk, kl in ((1, 40, 12, 0.0), (1, 40, 12, 1.0), (2, 40, 40, 1.0)):
        tokens, targets, bounds = data(base.vocab_size, B, L, seed=9)
        cfg = dataclasses.replace(base, index_kl_coef=kl, index_topk=topk)
        mine = fam.twin(cfg)
        fill(mine, 10)
        with torch.no_grad():
            for k, p in mine.state_dict().items():
                if k.endswith("router_bias"):
                    p.zero_()
        theirs = R.Dsv32(R.Dsv32Config(
            n_layers=cfg.n_layers, d_model=cfg.d_model, n_heads=cfg.n_heads, q_lora_rank=cfg.q_lora, kv_lora_rank=cfg.kv_lora,
            qk_nope_dim=cfg.d_nope, qk_rope_dim=cfg.d_rope, v_head_dim=cfg.d_v, first_k_dense=cfg.n_dense, d_ff_dense=cfg.d_ff,
            n_experts=cfg.n_experts, top_k=cfg.top_k, d_ff_expert=cfg.d_ff_expert, n_group=cfg.n_group, topk_group=cfg.topk_group,
            n_shared_experts=cfg.n_shared, d_ff_shared=cfg.n_shared * cfg.d_ff_expert, vocab_size=cfg.vocab_size,
            routed_scaling=cfg.routed_scaling, rope_base=cfg.rope_theta, index_n_heads=cfg.index_heads, index_head_dim=cfg.index_dim,
            index_topk=cfg.index_topk))
        pairs = {"embed.weight": I("wte"), "final_norm.weight": I("final_norm"), "lm_head.weight": T("w_head")}
        F_ = cfg.d_ff
        for i in range(cfg.n_layers):
            pairs.update(dsa_pairs(i))
            if i < cfg.n_dense:
                pairs.update({f"blocks.{i}.mlp.w1.weight": cols(f"layers.{i}.w13", 0, F_), f"blocks.{i}.mlp.w3.weight": cols(f"layers.{i}.w13", F_, 2 * F_),
                              f"blocks.{i}.mlp.w2.weight": T(f"layers.{i}.w2")})
            else:        # this module keeps the packed (in, out) orientation for its expert-side parameters
                pairs.update({f"blocks.{i}.mlp.w_router": I(f"layers.{i}.w_router"), f"blocks.{i}.mlp.w13_experts": I(f"layers.{i}.w13_experts"),
                              f"blocks.{i}.mlp.w2_experts": I(f"layers.{i}.w2_experts"), f"blocks.{i}.mlp.w_s13": I(f"layers.{i}.w13_shared"),
                              f"blocks.{i}.mlp.w_s2": I(f"layers.{i}.w2_shared"), f"blocks.{i}.mlp.w_router_bias": I(f"layers.{i}.router_bias")})

        def their_loss(m):
            if kl:
                for blk in m.blocks:
                    blk.attn.stash_idx_kl = True
            ce = m.loss(tokens.view(B, L), targets.view(B, L))
            if kl:       # the reported loss is the cross entropy; the indexer objective (KL summed over queries and layers,
                return ce, ce + kl * sum(blk.attn.idx_kl for blk in m.blocks)       # unscaled) only steers the indexer
            return ce
        check(mine, theirs, pairs, lambda m: m.loss(tokens, targets, bounds, total_rows=B * L), their_loss)


def test_glm52_twin_matches_the_reference_truth_tree():
    """Cross-layer index sharing with an irregular role pattern (a dense leader, a leader serving two followers, a leader
    serving nobody, a trailing short group): followers attend over their leader's selection, and the leader's indexer learns
    from the mean of the group's attention targets."""
    from dataflow_b200.models.families import resolve_family
    R = ref_module("glm52")
    fam = resolve_family("glm52")
    types = ("full", "full", "shared", "shared", "full", "shared")
    base = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32", rms_eps=1e-5, n_layers=6, n_dense=1, indexer_types=types)
    for B, L, topk, kl in ((1, 40, 12, 0.0), (1, 40, 12, 1.0), (2, 40, 40, 1.0)):
        tokens, targets, bounds = data(base.vocab_size, B, L, seed=13)
        cfg = dataclasses.replace(base, index_kl_coef=kl, index_topk=topk)
        mine = fam.twin(cfg)
        fill(mine, 14)
        with torch.no_grad():
            for k, p in mine.state_dict().items():
                if k.endswith("router_bias"):
                    p.zero_()
        theirs = R.Glm52(R.Glm52Config(
            n_layers=cfg.n_layers, d_model=cfg.d_model, n_heads=cfg.n_heads, q_lora_rank=cfg.q_lora, kv_lora_rank=cfg.kv_lora,
            qk_nope_dim=cfg.d_nope, qk_rope_dim=cfg.d_rope, v_head_dim=cfg.d_v, d_ff=cfg.d_ff, first_k_dense=cfg.n_dense,
            n_experts=cfg.n_experts, top_k=cfg.top_k, d_ff_expert=cfg.d_ff_expert, n_group=cfg.n_group, topk_group=cfg.topk_group,
            routed_scaling=cfg.routed_scaling, n_shared_experts=cfg.n_shared, d_ff_shared=cfg.n_shared * cfg.d_ff_expert,
            index_n_heads=cfg.index_heads, index_head_dim=cfg.index_dim, index_topk=cfg.index_topk, indexer_types=types,
            vocab_size=cfg.vocab_size, rope_base=cfg.rope_theta))
        pairs = {"embed.weight": I("wte"), "final_norm.weight": I("final_norm"), "lm_head.weight": T("w_head")}
        F_ = cfg.d_ff
        for i in range(cfg.n_layers):
            pairs.update(dsa_pairs(i) if types[i] == "full" else mla_pairs(i))
            if i < cfg.n_dense:
                pairs.update({f"blocks.{i}.ffn.w1.weight": cols(f"layers.{i}.w13", 0, F_), f"blocks.{i}.ffn.w3.weight": cols(f"layers.{i}.w13", F_, 2 * F_),
                              f"blocks.{i}.ffn.w2.weight": T(f"layers.{i}.w2")})
            else:
                pairs.update({f"blocks.{i}.ffn.w_router.weight": T(f"layers.{i}.w_router"), f"blocks.{i}.ffn.w13_experts": I(f"layers.{i}.w13_experts"),
                              f"blocks.{i}.ffn.w2_experts": I(f"layers.{i}.w2_experts"), f"blocks.{i}.ffn.w_s13.weight": T(f"layers.{i}.w13_shared"),
                              f"blocks.{i}.ffn.w_s2.weight": T(f"layers.{i}.w2_shared"), f"blocks.{i}.ffn.w_router_bias": I(f"layers.{i}.router_bias")})

        def their_loss(m):
            if kl:
                m.enable_indexer_kl(True)
            ce = m.loss(tokens.view(B, L), targets.view(B, L))
            return (ce, ce + kl * m.indexer_loss()) if kl else ce
        check(mine, theirs, pairs, lambda m: m.loss(tokens, targets, bounds, total_rows=B * L), their_loss)


def llama_like_pairs(d, i, their_mlp):
    """This repository packs [q | k | v] (and [gate | up]) into one field; the truth trees keep separate Linear layers."""
    L = f"layers.{i}."
    q, kv = d.n_heads * d.head_dim, d.n_kv_heads * d.head_dim
    p = {f"blocks.{i}.attn_norm.weight": I(L + "attn_norm"), f"blocks.{i}.ffn_norm.weight": I(L + "ffn_norm"),
         f"blocks.{i}.attn.wq.weight": cols(L + "w_qkv", 0, q), f"blocks.{i}.attn.wk.weight": cols(L + "w_qkv", q, q + kv),
         f"blocks.{i}.attn.wv.weight": cols(L + "w_qkv", q + kv, q + 2 * kv), f"blocks.{i}.attn.wo.weight": T(L + "wo")}
    if d.qk_norm:
        p.update({f"blocks.{i}.attn.q_norm.weight": I(L + "q_norm"), f"blocks.{i}.attn.k_norm.weight": I(L + "k_norm")})
    if d.n_experts:
        p.update({f"blocks.{i}.moe.w13_experts": I(L + "w13_experts"), f"blocks.{i}.moe.w2_experts": I(L + "w2_experts")})
        p.update({f"blocks.{i}.moe.router.weight": T(L + "w_router")} if their_mlp == "router_linear" else {f"blocks.{i}.moe.w_router": I(L + "w_router")})
    else:
        F_ = d.d_ff
        p.update({f"blocks.{i}.mlp.w1.weight": cols(L + "w13", 0, F_), f"blocks.{i}.mlp.w3.weight": cols(L + "w13", F_, 2 * F_),
                  f"blocks.{i}.mlp.w2.weight": T(L + "w2")})
    return p


def twin_loss(tokens, targets, bounds, rows):
    def f(m):
        logits = m(tokens, bounds)
        return torch.nn.functional.cross_entropy(logits.float(), targets.long(), reduction="sum") / rows
    return f


@pytest.mark.parametrize("family,cls,router", [("llama3", "Llama3", None), ("qwen3", "Qwen3", None), ("qwen3moe", "Qwen3Moe", "param"),
                                               ("olmoe", "Olmoe", "router_linear")])
def test_llama_like_twins_match_the_reference_truth_trees(family, cls, router):
    """Grouped-query attention with rotate-half RoPE and a SwiGLU MLP (llama3); RMSNorm on every head of q and k (qwen3); the
    mixture-of-experts MLP with top-k-then-softmax routing (qwen3moe); RMSNorm over the whole q / k row and
    softmax-then-top-k routing (olmoe).  Uniform and packed (ragged) rounds."""
    from dataflow_b200.models.families import resolve_family
    R = ref_module(family)
    fam = resolve_family(family)
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32")
    mine = fam.twin(cfg)
    fill(mine, 21)
    kw = dict(n_layers=cfg.n_layers, d_model=cfg.d_model, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, vocab_size=cfg.vocab_size,
              rope_base=cfg.rope_theta)
    if family != "llama3":
        kw["head_dim"] = cfg.head_dim
    kw.update(dict(n_experts=cfg.n_experts, top_k=cfg.top_k, d_ff_expert=cfg.d_ff_expert) if cfg.n_experts else dict(d_ff=cfg.d_ff))
    theirs = getattr(R, cls)(getattr(R, cls + "Config")(**kw))
    pairs = {"embed.weight": I("wte"), "final_norm.weight": I("final_norm"), "lm_head.weight": T("w_head")}
    for i in range(cfg.n_layers):
        pairs.update(llama_like_pairs(cfg, i, router))
    B, L = 2, 48
    tokens, targets, bounds = data(cfg.vocab_size, B, L, seed=22)
    check(mine, theirs, pairs, twin_loss(tokens, targets, bounds, B * L), lambda m: m.loss(tokens.view(B, L), targets.view(B, L)))
    ragged = [0, 17, 60, 96]
    lens = tuple(b - a for a, b in zip(ragged[:-1], ragged[1:]))
    mine.zero_grad()
    theirs.zero_grad()
    check(mine, theirs, pairs, twin_loss(tokens, targets, ragged, B * L),
          lambda m: m.loss(tokens.view(1, -1), targets.view(1, -1), seq_lens=lens))


@pytest.mark.parametrize("tied", [False, True])
def test_gpt2_twin_matches_the_reference_truth_tree(tied):
    """LayerNorm with bias, learned positions that restart in every packed sequence, fused qkv projection, tanh-GELU MLP, tied or
    untied head."""
    from dataflow_b200.models.families import resolve_family
    R = ref_module("gpt2")
    fam = resolve_family("gpt2")
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32", tied_embeddings=tied)
    mine = fam.twin(cfg)
    fill(mine, 31)
    theirs = R.Gpt2(R.Gpt2Config(n_layers=cfg.n_layers, d_model=cfg.d_model, n_heads=cfg.n_heads, d_ff=4 * cfg.d_model,
                                 vocab_size=cfg.vocab_size, n_ctx=cfg.max_positions, tied=tied, use_bias=True))
    pairs = {"wte.weight": I("wte"), "wpe.weight": I("wpe"), "final_norm.weight": I("final_norm"), "final_norm.bias": I("final_norm_b")}
    if not tied:
        pairs["lm_head.weight"] = T("w_head")
    for i in range(cfg.n_layers):
        L, B_ = f"layers.{i}.", f"blocks.{i}."
        pairs.update({B_ + "attn_norm.weight": I(L + "ln1_w"), B_ + "attn_norm.bias": I(L + "ln1_b"),
                      B_ + "attn.c_attn.weight": T(L + "c_attn_w"), B_ + "attn.c_attn.bias": I(L + "c_attn_b"),
                      B_ + "attn.c_proj.weight": T(L + "attn_proj_w"), B_ + "attn.c_proj.bias": I(L + "attn_proj_b"),
                      B_ + "ffn_norm.weight": I(L + "ln2_w"), B_ + "ffn_norm.bias": I(L + "ln2_b"),
                      B_ + "mlp.c_fc.weight": T(L + "fc_w"), B_ + "mlp.c_fc.bias": I(L + "fc_b"),
                      B_ + "mlp.c_proj.weight": T(L + "mlp_proj_w"), B_ + "mlp.c_proj.bias": I(L + "mlp_proj_b")})
    B, L_ = 2, 40
    tokens, targets, bounds = data(cfg.vocab_size, B, L_, seed=32)
    check(mine, theirs, pairs, lambda m: m.loss(tokens, targets, bounds, total_rows=B * L_),
          lambda m: m.loss(tokens.view(B, L_), targets.view(B, L_)))
    ragged = [0, 11, 50, 80]
    mine.zero_grad()
    theirs.zero_grad()
    check(mine, theirs, pairs, lambda m: m.loss(tokens, targets, ragged, total_rows=B * L_),
          lambda m: m.loss(tokens.view(1, -1), targets.view(1, -1), seq_lens=tuple(b - a for a, b in zip(ragged[:-1], ragged[1:]))))
