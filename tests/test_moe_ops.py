"""MoE routing / dispatch / grouped-GEMM ops: the eager lane against dense per-token math (CPU), and the sm_100a
kernels against the eager lane (GPU)."""
import pytest
import torch

from dataflow_b200.ops import eager as E


def dense_moe(x, logits, W, K, mode):
    w, ids = E.moe_topk_softmax(logits, K, mode)
    out = torch.zeros(x.shape[0], W.shape[2])
    for t in range(x.shape[0]):
        for k in range(K):
            out[t] += w[t, k] * (x[t] @ W[ids[t, k]])
    return out


@pytest.mark.parametrize("mode", ["topk_then_softmax", "softmax_then_topk"])
def test_eager_pipeline_equals_dense_math(mode):
    torch.manual_seed(0)
    t, K, Ex, d, F = 50, 2, 6, 16, 8
    logits, x, W = torch.randn(t, Ex), torch.randn(t, d), torch.randn(Ex, d, F)
    w, ids = E.moe_topk_softmax(logits, K, mode)
    row_of, row_src, offp, tile_e, counts = E.moe_sort(ids, Ex, tile_rows=8)
    assert int(counts.sum()) == t * K and offp[-1] % 8 == 0 and (offp[1:] - offp[:-1] >= counts).all()
    xp = E.moe_dispatch(x, row_src)
    assert (xp[row_src < 0] == 0).all()
    E.MOE_TILE_ROWS, keep = 8, E.MOE_TILE_ROWS
    try:
        h = E.moe_grouped_mm(xp, W, tile_e)
    finally:
        E.MOE_TILE_ROWS = keep
    y = E.moe_combine(None, h, w, row_of)
    assert torch.allclose(y, dense_moe(x, logits, W, K, mode), atol=1e-5)


def test_ties_go_to_the_smallest_index_and_order_is_stable():
    logits = torch.tensor([[1.0, 3.0, 3.0, 0.0], [2.0, 2.0, 2.0, 2.0]])
    _, ids = E.moe_topk_softmax(logits, 2)
    assert ids.tolist() == [[1, 2], [0, 1]]
    row_of, row_src, offp, _, _ = E.moe_sort(torch.tensor([[1, 0], [1, 0], [0, 1]], dtype=torch.int32), 2, tile_rows=4)
    assert row_src[:3].tolist() == [0, 1, 2] and row_src[4:7].tolist() == [0, 1, 2]      # token order inside an expert


@pytest.mark.parametrize("mode", ["topk_then_softmax", "softmax_then_topk"])
def test_router_backward_matches_autograd(mode):
    torch.manual_seed(1)
    logits = torch.randn(12, 8, requires_grad=True)
    w, ids = E.moe_topk_softmax(logits.detach(), 3, mode)
    # differentiable re-computation with the same selection
    if mode == "topk_then_softmax":
        wa = torch.softmax(logits.gather(1, ids.long()), -1)
    else:
        wa = torch.softmax(logits, -1).gather(1, ids.long())
    dp = torch.randn(12, 3)
    (wa * dp).sum().backward()
    got = E.moe_router_bwd(dp, w, ids, logits.detach(), mode)
    assert torch.allclose(got, logits.grad, atol=1e-6)


def test_sigmoid_noaux_grouped_selection():
    torch.manual_seed(2)
    logits, bias = torch.randn(20, 16), torch.zeros(16)
    w, ids = E.moe_topk_sigmoid_noaux(logits, bias, top_k=4, n_group=4, topk_group=2, routed_scaling=2.5)
    assert ((ids // 4).unique(dim=1).shape[1] <= 4) and all(len(set((r // 4).tolist())) <= 2 for r in ids)
    assert torch.allclose(w.sum(-1), torch.full((20,), 2.5), atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["topk_then_softmax", "softmax_then_topk"])
def test_gpu_router_and_data_movement_match_eager(mode):
    from dataflow_b200.ops import cuda as C
    torch.manual_seed(3)
    t, K, Ex, d = 3000, 8, 64, 512
    logits = torch.randn(t, Ex, device="cuda").bfloat16()
    w, ids = C.moe_topk_softmax(logits, K, mode)
    we, ide = E.moe_topk_softmax(logits, K, mode)
    assert torch.equal(ids, ide) and torch.allclose(w, we, atol=2e-6)
    dp = torch.randn(t, K, device="cuda")
    assert torch.allclose(C.moe_router_bwd(dp, w, ids, logits, mode), E.moe_router_bwd(dp, we, ide, logits, mode), atol=2e-6)
    row_of, row_src, offp, tile_e, counts = E.moe_sort(ids, Ex)
    x = torch.randn(t, d, device="cuda").bfloat16()
    xp = C.moe_dispatch(x, row_src)
    assert torch.equal(xp, E.moe_dispatch(x, row_src))
    base = torch.randn(t, d, device="cuda").bfloat16()
    assert torch.allclose(C.moe_combine(base, xp, w, row_of).float(), E.moe_combine(base, xp, we, row_of).float(), atol=2e-2, rtol=1e-2)
    assert torch.allclose(C.moe_dispatch_bwd(xp, row_of).float(), E.moe_dispatch_bwd(xp, row_of).float(), atol=2e-2, rtol=1e-2)
    assert torch.allclose(C.moe_rowdot(xp, xp, row_of), E.moe_rowdot(xp, xp, row_of), rtol=1e-3, atol=1e-2)
    a, b = xp.clone(), xp.clone()
    assert torch.allclose(C.moe_scale_rows(a, w, row_of).float(), E.moe_scale_rows(b, we, row_of).float(), atol=1e-2, rtol=1e-2)


@pytest.mark.gpu
def test_gpu_grouped_gemms_match_eager():
    from dataflow_b200.ops import cuda as C, native
    torch.manual_seed(4)
    t, K, Ex, d, F = 4096, 8, 16, 512, 256
    ids = E.moe_topk_softmax(torch.randn(t, Ex, device="cuda"), K)[1]
    ids[:, 0] = ids[:, 0].clamp(max=Ex - 2)                 # leave the last expert rare but present
    row_of, row_src, offp, tile_e, counts = E.moe_sort(ids, Ex)
    x = (torch.randn(t, d, device="cuda") * 0.5).bfloat16()
    xp = C.moe_dispatch(x, row_src)
    W = (torch.randn(Ex, d, 2 * F, device="cuda") * 0.05).bfloat16()
    h = C.moe_grouped_mm(xp, W, tile_e)
    torch.cuda.synchronize()
    assert native().gemm_last_error() == 0
    ref = E.moe_grouped_mm(xp, W, tile_e)
    used = int(offp[-1])                    # row tiles past the last expert are skipped by the kernel: never read
    assert ((h[:used].float() - ref[:used].float()).norm() / ref.float().norm()) < 5e-3
    h[used:].zero_()
    # dgrad through the transpose: (Mp, 2F) x W^T -> (Mp, d)
    dx = C.moe_grouped_mm(h, W, tile_e, transpose_w=True)
    refd = E.moe_grouped_mm(h, W, tile_e, transpose_w=True)
    assert ((dx[:used].float() - refd[:used].float()).norm() / refd.float().norm()) < 5e-3
    # wgrad, create then accumulate
    dW = torch.full_like(W, float("nan"))
    C.moe_grouped_wgrad(xp, h, offp, dW, accumulate=False)
    refw = E.moe_grouped_wgrad(xp, h, offp, torch.zeros_like(W), accumulate=False)
    torch.cuda.synchronize()
    assert native().gemm_last_error() == 0
    assert ((dW.float() - refw.float()).norm() / refw.float().norm()) < 5e-3
    C.moe_grouped_wgrad(xp, h, offp, dW, accumulate=True)
    assert ((dW.float() - 2 * refw.float()).norm() / (2 * refw.float()).norm()) < 8e-3


@pytest.mark.gpu
@pytest.mark.parametrize("t,n_experts,k", [(1, 4, 2), (700, 64, 8), (5000, 8, 2), (16384, 64, 8), (333, 256, 8), (100, 16, 1)])
def test_gpu_moe_sort_equals_the_stable_sort_oracle(t, n_experts, k):
    """The device counting sort (three kernels) gives exactly the eager layout: the same row for every slot (stable within an
    expert), the same source tokens, padded offsets, per-tile experts and counts; skewed routing included."""
    from dataflow_b200.ops import resolve_kernels
    K = resolve_kernels()
    g = torch.Generator(device="cuda").manual_seed(t)
    ids = torch.stack([torch.randperm(n_experts, device="cuda", generator=g)[:k] for _ in range(min(t, 64))])
    ids = ids[torch.randint(0, ids.shape[0], (t,), device="cuda", generator=g)].to(torch.int32)
    if t > 100:
        ids[: t // 2, 0] = 0                              # half of the tokens pile onto expert 0
    got = K.moe_sort(ids, n_experts)
    want = E.moe_sort(ids, n_experts)
    for a, b, name in zip(got, want, ("row_of", "row_src", "offsets_pad", "tile_expert", "counts")):
        assert a.dtype == torch.int32 and torch.equal(a, b.to(a.device)), name
