"""dsv3, dsv32, glm52, qwen35, qwen35moe: families in the reference-form (autograd) lane against their twins."""
import pytest
import torch

from dataflow_b200.models import _forms as F
from dataflow_b200.models.families import resolve_family, validate_family
from dataflow_b200.testing.family_gate import run_pair

FAMILIES = ["dsv3", "dsv32", "glm52", "qwen35", "qwen35moe"]


@pytest.mark.parametrize("family", FAMILIES)
def test_family_structure(family):
    assert validate_family(family) == []
    fam = resolve_family(family)
    cfg = fam.presets["tiny"]()
    prog = fam.lower(cfg)
    kinds = fam.derive_dims(cfg).kinds
    assert len(set(kinds)) >= 2                                    # every one of these stacks mixes kinds of layers
    for i, kind in enumerate(kinds):
        assert any(t.compute_block_key == f"{kind}_fwd" and t.block_params["layer"] == i for t in prog.tasks)
    lay = fam.family_layouts(fam.derive_dims(cfg))
    sizes = prog.object_sizes()
    for i in range(cfg.n_layers):
        assert sizes[f"W_{i}"] == lay.of_layer(i)[0].size_bytes


@pytest.mark.parametrize("family", FAMILIES)
def test_engine_matches_twin_fp32(family):
    r = run_pair(family, steps=3)
    assert r["max_loss_rel"] < 1e-3
    assert r["engine"][-1] < r["engine"][0]


@pytest.mark.parametrize("family", ["dsv32", "qwen35"])
def test_ragged_rounds_match_twin(family):
    assert run_pair(family, steps=2, shape="ragged")["max_loss_rel"] < 1e-3


def test_glm52_followers_read_their_leaders_selection_and_budget_does_not_change_losses():
    fam = resolve_family("glm52")
    cfg = fam.presets["tiny"]()
    prog = fam.lower(cfg)
    kinds = fam.derive_dims(cfg).kinds
    assert kinds == ("gdl", "gdf", "gml", "gmf")
    for t in prog.tasks:
        if t.compute_block_key in ("gdf_fwd", "gdf_bwd", "gmf_fwd", "gmf_bwd"):
            r, i = t.block_params["round"], t.block_params["layer"]
            assert f"A_0_{r}_{i - 1}" in t.inputs
        if t.compute_block_key in ("gdl_fwd", "gml_bwd"):
            assert sum(x.startswith("A_") for x in t.inputs) <= 1
    lay = fam.family_layouts(fam.derive_dims(cfg))
    assert "wi_q" in lay.of_layer(0)[0].names() and "wi_q" not in lay.of_layer(1)[0].names()
    free = run_pair("glm52", steps=2)
    tight = run_pair("glm52", steps=2, budget_gib=0.012)
    assert tight["engine"] == pytest.approx(free["engine"], rel=1e-6)


def test_dsv32_dense_warmup_trains_the_indexer_and_nothing_else():
    """Warm-up: dense attention, KL of the indexer to the full-prefix attention distribution, updates for ``wi_*`` only."""
    res = run_pair("dsv32", steps=3, preset="tiny_warmup")
    assert res["max_loss_rel"] < 1e-3
    moved = {k: v for k, v in res["weight_rel_l2"].items()}
    fam = resolve_family("dsv32")
    cfg = fam.presets["tiny_warmup"]()
    assert cfg.trainable_patterns == ("wi_*",)
    # the engine's final weights against ITS OWN initial weights: only the indexer moved
    import dataclasses
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    c32 = dataclasses.replace(cfg, dtype_policy="fp32")
    tr = Trainer("dsv32", c32, budget_gib=None, device=None, hyper={"lr": 2e-3, "weight_decay": 0.1}, seed=3)
    before = fam.bridge(c32, tr.views_of)
    losses = [tr.step(synthetic_rounds(c32, tr.rounds, tr.T, 64, 11, 0)) for _ in range(2)]        # the same batch twice
    tr.sync_to_host()
    after = fam.bridge(c32, tr.views_of)
    tr.close()
    changed = {k for k in before if not torch.equal(before[k], after[k])}
    assert changed and all(".wi_" in k for k in changed)
    assert {k.rsplit(".", 1)[-1] for k in changed} == {"wi_q", "wi_k", "wi_k_gain", "wi_k_bias", "wi_w"}
    assert abs(losses[1] - losses[0]) < 1e-6        # dense attention does not see the indexer: a frozen main model repeats its loss
    # dense attention: the sparse preset and the warm-up preset differ in their forward
    sparse = run_pair("dsv32", steps=1)["engine"][0]
    assert abs(sparse - res["engine"][0]) > 1e-7


def test_glm52_indexer_target_sums_over_the_group():
    """Groups of three: the last member's backward creates the accumulator, the middle one mutates it, the leader's reads
    it; the engine and the twin (which collects the followers' targets in a first pass) train the indexer alike."""
    fam = resolve_family("glm52")
    over = {"index_share": 3, "n_layers": 6, "n_dense": 2}
    import dataclasses
    cfg = dataclasses.replace(fam.presets["tiny"](), **over)
    prog = fam.lower(cfg)
    assert fam.derive_dims(cfg).kinds == ("gdl", "gdf", "gmf", "gml", "gmf", "gmf")
    by = {(t.block_params["layer"], t.block_params["round"]): t for t in prog.tasks
          if (t.compute_block_key or "").endswith("_bwd") and "layer" in t.block_params}
    for r in range(cfg.grad_accum_rounds):
        for lead in (0, 3):
            gid = f"G_0_{r}_{lead}"
            assert gid in [o.id for o in by[(lead + 2, r)].outputs]
            assert gid in by[(lead + 1, r)].mutates and gid in by[(lead, r)].inputs
    assert prog.object_sizes()["G_0_0_0"] == 4 * cfg.seq_len * cfg.batch * min(cfg.index_topk, cfg.seq_len)
    res = run_pair("glm52", steps=3, overrides=over)
    assert res["max_loss_rel"] < 1e-3
    # three AdamW steps amplify rounding differences into a few percent of weight distance in every field of this gate;
    # an engine that left the followers' share out lands at 0.16 - 0.17 on these four fields
    idx = {k: v for k, v in res["weight_rel_l2"].items() if k.endswith((".wi_q", ".wi_k"))}
    assert len(idx) == 4 and max(idx.values()) < 0.05
    # the followers' share moves the leader's auxiliary loss
    from dataflow_b200.data.segments import make_segments
    from dataflow_b200.models.glm52 import block_fn, kind_fields
    c = fam.presets["tiny"]()
    g = torch.Generator().manual_seed(0)
    n = c.seq_len
    w = {f.name: torch.randn(tuple(f.shape), generator=g) * (0.3 if len(f.shape) > 1 else 1.0) for f in kind_fields(c, "gdl")}
    x = torch.randn(n, c.d_model, generator=g)
    seg = make_segments([0, n], None)
    _, aux_own, emit = block_fn(c, "gdl", x, w, seg, 0)
    wf = {k: v for k, v in w.items() if not k.startswith("wi_")}
    _, aux_f, emit_f = block_fn(c, "gdf", torch.randn(n, c.d_model, generator=g), wf, seg, 1, shared=emit)
    assert aux_f is None and set(emit_f) == {"_deposit"}
    dep = emit_f["_deposit"]["kl_target"]
    assert dep.shape == (n, min(c.index_topk, c.seq_len)) and torch.allclose(dep.sum(-1), torch.ones(n), atol=1e-4)
    _, aux_group, _ = block_fn(c, "gdl", x, w, seg, 0, accum=emit_f["_deposit"], group_size=2)
    assert abs(float(aux_group) - float(aux_own)) > 1e-6


def test_delta_rule_with_full_write_strength_stores_and_recalls_an_association():
    # one head, orthonormal keys, beta = 1, no decay: after writing (k_i -> v_i) the state returns v_i for q = k_i
    dk = dv = 4
    k = torch.eye(dk)[:3].view(3, 1, dk)
    v = torch.randn(3, 1, dv)
    g, beta = torch.zeros(3, 1), torch.ones(3, 1)
    start = torch.zeros(3, dtype=torch.long)
    o = F.gated_delta_rule(k * dk ** 0.5, k, v, g, beta, start)      # the rule scales q by dk^-0.5
    assert torch.allclose(o, v, atol=1e-5)
    # a second write to the same key REPLACES the value (delta rule), it does not add to it
    k2 = torch.stack([k[0], k[0]]);  v2 = torch.randn(2, 1, dv)
    o2 = F.gated_delta_rule(k2 * dk ** 0.5, k2, v2, torch.zeros(2, 1), torch.ones(2, 1), torch.zeros(2, dtype=torch.long))
    assert torch.allclose(o2[1], v2[1], atol=1e-5)
    # a segment start clears the state
    o3 = F.gated_delta_rule(k2 * dk ** 0.5, k2, v2, torch.zeros(2, 1), torch.zeros(2, 1) + 1e-9, torch.tensor([0, 1]))
    assert o3[1].abs().max() < 1e-6


def test_causal_conv_never_reads_across_a_segment_start():
    x = torch.randn(10, 3)
    w = torch.randn(3, 4)
    start = torch.tensor([0] * 6 + [6] * 4)
    full = F.causal_conv1d_silu(x, w, start)
    tail = F.causal_conv1d_silu(x[6:], w, torch.zeros(4, dtype=torch.long))
    assert torch.allclose(full[6:], tail, atol=1e-6)


def test_sigmoid_noaux_routing_restricts_selection_to_the_best_groups():
    logits = torch.tensor([[5.0, 4.0, -9.0, -9.0, 3.0, 3.5, 3.6, 3.7]])
    w, ids = F.route_sigmoid_noaux(logits, torch.zeros(8), k=2, n_group=2, topk_group=1, scaling=2.0)
    assert set(ids[0].tolist()) == {0, 1}                             # group 0 has the larger sum of its two best scores
    assert w.sum().item() == pytest.approx(2.0, rel=1e-5)
    # one very good expert does not carry its group: the rank is the sum of the two best
    lone = torch.tensor([[9.0, -9.0, -9.0, -9.0, 2.0, 2.0, 2.0, 2.0]])
    _, ids1 = F.route_sigmoid_noaux(lone, torch.zeros(8), k=2, n_group=2, topk_group=1, scaling=1.0)
    assert set(ids1[0].tolist()) <= {4, 5, 6, 7}
    w2, ids2 = F.route_sigmoid_noaux(logits, torch.tensor([0, 0, 0, 0, 0, 0, 0, -10.0]), 2, 1, 1, 1.0)
    assert 7 not in ids2[0].tolist()                                  # the bias steers selection ...
    assert w2.sum().item() == pytest.approx(1.0, rel=1e-5)            # ... the weights come from the unbiased scores


def test_dsa_topk_mask_keeps_k_visible_keys_per_query():
    torch.manual_seed(0)
    n = 12
    causal = torch.tril(torch.ones(n, n, dtype=torch.bool))
    m = F.dsa_topk_mask(torch.randn(n, n), causal, 4)
    assert (m & ~causal).sum() == 0
    assert m.sum(-1).tolist() == [min(i + 1, 4) for i in range(n)]


@pytest.mark.gpu
@pytest.mark.parametrize("family", FAMILIES)
def test_gpu_engine_in_band(family):
    r = run_pair(family, device=0, policy="bf16_master", steps=3)
    assert r["max_loss_rel"] < 3e-2
    assert r["engine"][-1] < r["engine"][0]


@pytest.mark.parametrize("bounds", [[0, 200], [0, 37, 101, 300], [0, 128, 256]])
def test_chunked_gated_delta_rule_matches_the_sequential_form(bounds):
    """The chunk-parallel delta rule (triangular solve per chunk, only the state crosses chunk borders) against the
    token-by-token recurrence: outputs and all five gradients, uniform and ragged rounds, lengths that are not a multiple
    of the chunk."""
    torch.manual_seed(3)
    n, h, dk, dv = bounds[-1], 3, 16, 24
    q = torch.nn.functional.normalize(torch.randn(n, h, dk), dim=-1).requires_grad_()
    k = torch.nn.functional.normalize(torch.randn(n, h, dk), dim=-1).requires_grad_()
    v = torch.randn(n, h, dv, requires_grad=True)
    g = (-torch.rand(n, h) * 0.3).requires_grad_()
    beta = torch.rand(n, h).requires_grad_()
    seg = torch.zeros(n, dtype=torch.long)
    for a, b in zip(bounds[:-1], bounds[1:]):
        seg[a:b] = a
    o_seq = F.gated_delta_rule_sequential(q, k, v, g, beta, seg)
    o_chk = F.gated_delta_rule(q, k, v, g, beta, seg, chunk=32)
    assert torch.allclose(o_chk, o_seq, atol=2e-6, rtol=1e-5)
    w = torch.randn_like(o_seq)
    for a, b in zip(torch.autograd.grad((o_seq * w).sum(), [q, k, v, g, beta]), torch.autograd.grad((o_chk * w).sum(), [q, k, v, g, beta])):
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)


def test_dsa_gathered_forms_equal_the_masked_forms():
    """Long-context sparse attention (chunked index scores -> top-k rows, latent-form attention over the gathered keys, KL at the
    selection) gives the loss and every gradient of the (n, n)-mask forms; uniform and ragged rounds, chunks smaller than a
    sequence."""
    import dataclasses
    from dataflow_b200.models import _forms as F
    from dataflow_b200.data.segments import make_segments
    g = torch.Generator().manual_seed(5)
    B, L = 2, 40
    for family, bounds in (("dsv32", [0, 40, 80]), ("dsv32", [0, 13, 51, 80]), ("glm52", [0, 13, 51, 80])):
        fam = resolve_family(family)          # glm52: followers read the leader's published rows, targets flow back to it
        base = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32", index_topk=12, index_kl_coef=1.0)
        tokens = torch.randint(0, base.vocab_size, (B * L,), generator=g)
        targets = torch.randint(0, base.vocab_size, (B * L,), generator=g)
        got = {}
        for impl in ("mask", "gather"):
            m = fam.twin(dataclasses.replace(base, sparse_impl=impl))
            gg = torch.Generator().manual_seed(3)
            with torch.no_grad():
                for p in m.parameters():
                    p.copy_(torch.randn(p.shape, generator=gg) * (p.shape[-2] ** -0.5 if p.dim() > 1 else 0.1) + (1.0 if p.dim() == 1 else 0.0))
            loss = m.loss(tokens, targets, bounds, total_rows=B * L)
            loss.backward()
            got[impl] = (loss.item(), {k: p.grad for k, p in m.named_parameters()})
        assert got["mask"][0] == pytest.approx(got["gather"][0], rel=1e-6)
        for k, ga in got["mask"][1].items():
            gb = got["gather"][1][k]
            assert (ga is None) == (gb is None), k
            if ga is not None:
                assert float((ga - gb).norm() / (ga.norm() + 1e-12)) < 1e-4, k
    # the chunked pieces against their dense counterparts, chunks of 16 queries
    c = base
    n = 80
    seg = make_segments([0, 13, 51, 80], None)
    pos = seg.positions[:n]
    x, cq = torch.randn(n, c.d_model, generator=g), torch.randn(n, c.q_lora or c.d_model, generator=g)
    w = {k: torch.randn(s, generator=g) * 0.2 for k, s in (("wi_q", (cq.shape[1], c.index_heads * c.index_dim)), ("wi_k", (c.d_model, c.index_dim)),
                                                         ("wi_k_gain", (c.index_dim,)), ("wi_k_bias", (c.index_dim,)), ("wi_w", (c.d_model, c.index_heads)))}
    causal = F.segment_causal_mask(seg, n, x.device)
    dense = F.dsa_index_scores(x, cq, w, c, pos)
    sel, live = F.dsa_select(x, cq, w, c, pos, 12, chunk=16)
    want = F.dsa_topk_mask(dense, causal, 12)
    have = torch.zeros_like(causal)
    have[torch.arange(n)[:, None].expand_as(sel)[live], sel[live]] = True
    # ReLU leaves exact zeros, and which of several tied keys a top-k keeps is the library's business: the two selections must
    # agree as multisets of scores, row by row
    assert torch.equal(have.sum(1), want.sum(1))
    a = dense.masked_fill(~have, float("-inf")).sort(dim=1, descending=True).values[:, :12]
    b = dense.masked_fill(~want, float("-inf")).sort(dim=1, descending=True).values[:, :12]
    assert torch.allclose(a, b, atol=1e-6)
    at = F.dsa_scores_at(x, cq, w, c, pos, sel)
    assert torch.allclose(at[live], dense.gather(1, sel)[live], atol=1e-5)


@pytest.mark.gpu
def test_dsv32_trains_a_step_at_sequence_16384_on_one_gpu():
    """Long context on the sparse lane: full-size indexer (64 heads of 128, top-2048) at 16 384 tokens.  The index scores run on
    the tensor cores, the selection in the radix kernel, attention over the gathered keys in the latent form; nothing of size
    (n, n) is ever allocated (the dense forms would need 68 GB of probabilities per layer)."""
    import dataclasses
    import time
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    fam = resolve_family("dsv32")
    cfg = dataclasses.replace(fam.presets["dsv32_long16k"](), n_layers=2)
    torch.cuda.reset_peak_memory_stats()
    tr = Trainer("dsv32", cfg, budget_gib=40.0, device=0, hyper={"lr": 1e-3, "weight_decay": 0.0}, seed=1)
    losses = []
    t0 = time.perf_counter()
    for s in range(2):
        losses.append(tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, cfg.vocab_size, 5, s)))
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / 2
    peak = torch.cuda.max_memory_allocated() / 2 ** 30
    tr.close()
    print(f"dsv32 long context: {dt:.2f} s per step of {cfg.seq_len} tokens, framework allocator peak {peak:.1f} GiB, losses {losses}")
    assert all(l == l and 0 < l < 20 for l in losses)
    assert peak < 64.0          # the dense forms hold 32 heads x 16384^2 fp32 probabilities = 34 GB per layer, twice with their gradient
