"""Write-coverage battery: every native op, on a regular and on a degenerate geometry, run twice over differently
poisoned memory must return the same bytes — an output element the kernel forgets to write (a tail row, the last partial
tile, a padding slot) shows up as poison that differs between the runs.  Ops allocate most outputs themselves, so the
poison goes into the caching allocator's free blocks: fill, free, and the next ``torch.empty`` hands the poisoned bytes back.

The case table is keyed by op name and must name every native op (tripwire, CPU).  Each case also runs against the eager
lane on CPU (no GPU needed), which keeps the table's calls valid where no device is present.
Parity: reference ``tests/dataflow_training/tasks/test_kernel_audit.py`` (double-run poison coverage, degenerate geometry,
completeness tripwire).
"""
import pytest
import torch

from dataflow_b200.ops import registered_ops, resolve_kernels

BF, F32, I32 = torch.bfloat16, torch.float32, torch.int32


class G:
    """Random inputs on one device from one seed."""

    def __init__(self, dev, seed=0):
        self.dev = dev
        self.g = torch.Generator(device=dev).manual_seed(seed)

    def bf(self, *shape, scale=1.0):
        return (torch.randn(*shape, device=self.dev, generator=self.g) * scale).to(BF)

    def f32(self, *shape, scale=1.0):
        return torch.randn(*shape, device=self.dev, generator=self.g) * scale

    def ints(self, hi, *shape):
        return torch.randint(0, hi, shape, device=self.dev, generator=self.g).to(I32)


def seg_tables(g, lens):
    n = sum(lens)
    bounds = [0]
    for l in lens:
        bounds.append(bounds[-1] + l)
    cu = torch.tensor(bounds, dtype=I32, device=g.dev)
    pos = torch.cat([torch.arange(l, dtype=I32) for l in lens]).to(g.dev)
    start = torch.cat([torch.full((l,), b, dtype=I32) for l, b in zip(lens, bounds)]).to(g.dev)
    return n, cu, pos, start, max(lens)


def moe_tables(K, g, t, E, topk):
    ids = torch.stack([torch.randperm(E, device=g.dev, generator=g.g)[:topk] for _ in range(t)]).to(I32)
    return (ids,) + tuple(K.moe_sort(ids, E))


# geometry: (rows, cols) pairs; "odd" stresses tails (rows not a multiple of any tile, one row, minimum width)
def dims(small):
    return (1, 64) if small else (333, 768)


def c_rmsnorm_fwd(K, g, small):
    r, c = dims(small)
    return K.rmsnorm_fwd(g.bf(r, c), g.bf(c) + 1, 1e-5)


def c_rmsnorm_apply(K, g, small):
    r, c = dims(small)
    return K.rmsnorm_apply(g.bf(r, c), g.bf(c) + 1, g.f32(r).abs() + 0.5)


def c_rmsnorm_bwd(K, g, small):
    r, c = dims(small)
    dw = torch.zeros(c, device=g.dev, dtype=F32)
    dx = K.rmsnorm_bwd(g.bf(r, c), g.bf(r, c), g.bf(c) + 1, g.f32(r).abs() + 0.5, dx_add=g.bf(r, c), dw=dw, accumulate=False)
    return dx, dw


def c_layernorm_fwd(K, g, small):
    r, c = dims(small)
    return K.layernorm_fwd(g.bf(r, c), g.bf(c) + 1, g.bf(c), 1e-5)


def c_layernorm_apply(K, g, small):
    r, c = dims(small)
    return K.layernorm_apply(g.bf(r, c), g.bf(c) + 1, g.bf(c), g.f32(r), g.f32(r).abs() + 0.5)


def c_layernorm_bwd(K, g, small):
    r, c = dims(small)
    dw, db = torch.zeros(c, device=g.dev, dtype=F32), torch.zeros(c, device=g.dev, dtype=F32)
    dx = K.layernorm_bwd(g.bf(r, c), g.bf(r, c), g.bf(c) + 1, g.f32(r), g.f32(r).abs() + 0.5, dw=dw, db=db, accumulate=False)
    return dx, dw, db


def c_rope(fn):
    def case(K, g, small):
        n, cu, pos, start, mx = seg_tables(g, [1] if small else [37, 200, 96])
        x = g.bf(n, 3, 128)
        getattr(K, fn)(x, pos, 10000.0)
        return x
    return case


def attn_inputs(g, small):
    n, cu, pos, start, mx = seg_tables(g, [1] if small else [130, 257, 64])
    return n, cu, mx, g.bf(n, 4, 128, scale=0.5), g.bf(n, 2, 128, scale=0.5), g.bf(n, 2, 128, scale=0.5)


def c_flash_fwd(K, g, small):
    n, cu, mx, q, k, v = attn_inputs(g, small)
    return K.flash_fwd(q, k, v, cu, mx)


def c_flash_bwd(K, g, small):
    n, cu, mx, q, k, v = attn_inputs(g, small)
    out, lse = K.flash_fwd(q, k, v, cu, mx)
    return K.flash_bwd(g.bf(n, 4, 128), q, k, v, out, lse, cu, mx)


def c_swiglu_fwd_out(K, g, small):
    r, c = dims(small)
    h = g.bf(r, 2 * c)
    return K.swiglu_fwd_out(h[:, :c], h[:, c:])


def c_swiglu_bwd(K, g, small):
    r, c = dims(small)
    h = g.bf(r, 2 * c)
    return K.swiglu_bwd(g.bf(r, c), h[:, :c], h[:, c:])


def c_swiglu_packed_fwd(K, g, small):
    r, c = dims(small)
    return K.swiglu_packed_fwd(g.bf(r, 2 * c))


def c_swiglu_packed_bwd(K, g, small):
    r, c = dims(small)
    return K.swiglu_packed_bwd(g.bf(r, c), g.bf(r, 2 * c), with_s=True)


def c_gelu_fwd_out(K, g, small):
    r, c = dims(small)
    return K.gelu_fwd_out(g.bf(r, c))


def c_gelu_bwd(K, g, small):
    r, c = dims(small)
    return K.gelu_bwd(g.bf(r, c), g.bf(r, c))


def c_ce_loss(K, g, small):
    r, v = (1, 64) if small else (301, 1000)
    logits = g.bf(r, v)
    tg = g.ints(v, r)
    if not small:
        tg[::7] = -1
    loss = K.ce_loss_fwd_bwd(logits, tg, total_rows=r)
    return logits, loss


def c_embed_fwd(K, g, small):
    r, d, v = (1, 64, 8) if small else (300, 256, 1000)
    return K.embed_fwd(g.ints(v, r), g.bf(v, d))


def c_embed_bwd(K, g, small):
    r, d, v = (1, 64, 8) if small else (300, 256, 50)
    dt = torch.zeros(v, d, device=g.dev, dtype=BF)
    K.embed_bwd_accum(g.ints(v, r), g.bf(r, d), dt, accumulate=False)
    return dt


def c_adamw(K, g, small):
    n = 8 if small else 10007 * 8
    w, m, v = g.bf(n), torch.zeros(n, device=g.dev, dtype=BF), torch.zeros(n, device=g.dev, dtype=BF)
    K.adamw_step(w, g.bf(n), m, v, lr=1e-3, wd=0.1, step=3)
    return w, m, v


def c_adamw_split(K, g, small):
    n = 8 if small else 10007 * 8
    w, lo = g.bf(n), torch.zeros(n, device=g.dev, dtype=torch.int16)
    m, v = torch.zeros(n, device=g.dev, dtype=BF), torch.zeros(n, device=g.dev, dtype=BF)
    K.adamw_split_step(w, lo, g.bf(n), m, v, lr=1e-3, wd=0.1, step=3)
    return w, lo, m, v


def c_sgd(K, g, small):
    n = 8 if small else 10007
    w, m = g.bf(n), torch.zeros(n, device=g.dev, dtype=BF)
    K.sgd_step(w, g.bf(n), m, lr=0.05, momentum=0.9, wd=0.01)
    return w, m


def gemm_dims(small):
    return (1, 64, 64) if small else (300, 256, 328)


def c_linear_fwd(K, g, small):
    m, k, n = gemm_dims(small)
    return K.linear_fwd_bf16(g.bf(m, k, scale=0.1), g.bf(k, n, scale=0.1), add=g.bf(m, n), bias=g.bf(n))


def c_linear_dgrad(K, g, small):
    m, k, n = gemm_dims(small)
    return K.linear_dgrad_bf16(g.bf(m, n, scale=0.1), g.bf(k, n, scale=0.1))


def c_linear_wgrad(K, g, small):
    m, k, n = gemm_dims(small)
    dw = torch.zeros(k, n, device=g.dev, dtype=BF)
    K.linear_wgrad_bf16(g.bf(m, k, scale=0.1), g.bf(m, n, scale=0.1), dw, accumulate=False)
    return dw


def c_bias_grad(K, g, small):
    r, c = dims(small)
    db = torch.zeros(c, device=g.dev, dtype=BF)
    K.bias_grad(g.bf(r, c), db, accumulate=False)
    return db


def c_add(K, g, small):
    r, c = dims(small)
    return K.add(g.bf(r, c), g.bf(r, c))


def c_moe_sort(K, g, small):
    t, E, topk = (1, 4, 2) if small else (700, 64, 8)
    ids = torch.stack([torch.randperm(E, device=g.dev, generator=g.g)[:topk] for _ in range(t)]).to(I32)
    return K.moe_sort(ids, E)


def c_moe_topk_softmax(K, g, small):
    t, E = (1, 8) if small else (301, 64)
    return K.moe_topk_softmax(g.bf(t, E), 2, "topk_then_softmax")


def c_moe_topk_sigmoid(K, g, small):
    t, E = (1, 8) if small else (301, 64)
    return K.moe_topk_sigmoid_noaux(g.bf(t, E), g.f32(E, scale=0.01), 2, 4, 2, 2.5)


def c_moe_router_bwd(K, g, small):
    t, E = (1, 8) if small else (301, 64)
    logits = g.bf(t, E)
    w, ids = K.moe_topk_softmax(logits, 2, "topk_then_softmax")
    return K.moe_router_bwd(g.f32(t, 2), w, ids, logits, "topk_then_softmax")


def moe_case(fn):
    def case(K, g, small):
        t, E, topk, d = (1, 4, 2, 64) if small else (200, 8, 2, 128)
        ids, row_of, row_src, off, tile_e, counts = moe_tables(K, g, t, E, topk)
        return fn(K, g, t, E, topk, d, ids, row_of, row_src, off, tile_e)
    return case


def _dispatch(K, g, t, E, topk, d, ids, row_of, row_src, off, tile_e):
    return K.moe_dispatch(g.bf(t, d), row_src)


def _combine(K, g, t, E, topk, d, ids, row_of, row_src, off, tile_e):
    return K.moe_combine(g.bf(t, d), g.bf(row_src.numel(), d), g.f32(t, topk), row_of)


def _dispatch_bwd(K, g, t, E, topk, d, ids, row_of, row_src, off, tile_e):
    return K.moe_dispatch_bwd(g.bf(row_src.numel(), d), row_of)


def _scale_rows(K, g, t, E, topk, d, ids, row_of, row_src, off, tile_e):
    xp = g.bf(row_src.numel(), d)
    K.moe_scale_rows(xp, g.f32(t, topk), row_of)
    return xp


def _rowdot(K, g, t, E, topk, d, ids, row_of, row_src, off, tile_e):
    return K.moe_rowdot(g.bf(row_src.numel(), d), g.bf(row_src.numel(), d), row_of)


def _grouped_mm(K, g, t, E, topk, d, ids, row_of, row_src, off, tile_e):
    xp = K.moe_dispatch(g.bf(t, d, scale=0.2), row_src)
    # row tiles past the last expert's rows (tile_expert == -1) are nobody's: the op leaves them as they are
    return K.moe_grouped_mm(xp, g.bf(E, d, 2 * d, scale=0.1), tile_e)[: int(off[-1])]


def _grouped_wgrad(K, g, t, E, topk, d, ids, row_of, row_src, off, tile_e):
    xp = K.moe_dispatch(g.bf(t, d, scale=0.2), row_src)
    dyp = K.moe_dispatch(g.bf(t, 64, scale=0.2), row_src)
    dw = torch.zeros(E, d, 64, device=g.dev, dtype=BF)
    K.moe_grouped_wgrad(xp, dyp, off, dw, accumulate=False)
    return dw


def c_dsa_scores(K, g, small):
    n, cu, pos, start, mx = seg_tables(g, [1] if small else [100, 230])
    return K.dsa_index_scores(g.bf(n, 3, 64, scale=0.3), g.bf(n, 64, scale=0.3), g.f32(n, 3), start, 0, n, 0)


def c_dsa_topk(K, g, small):
    rows, cols, k = (1, 1, 4) if small else (37, 700, 64)
    s = torch.relu(g.f32(rows, cols))
    return K.dsa_topk_rows(s, k, 3)


def c_l2norm_fwd(K, g, small):
    r, c = (1, 64) if small else (333, 128)
    return K.l2norm_fwd(g.bf(r, c))


def c_l2norm_bwd(K, g, small):
    r, c = (1, 64) if small else (333, 128)
    return K.l2norm_bwd(g.bf(r, c), g.bf(r, c), g.f32(r).abs() + 0.5)


def c_gated_rmsnorm_fwd(K, g, small):
    r, c = (1, 64) if small else (333, 128)
    return K.gated_rmsnorm_fwd(g.bf(r, c), g.bf(r, c), g.bf(c) + 1)


def c_gated_rmsnorm_bwd(K, g, small):
    r, c = (1, 64) if small else (333, 128)
    return K.gated_rmsnorm_bwd(g.bf(r, c), g.bf(r, c), g.bf(r, c), g.bf(c) + 1, g.f32(r).abs() + 0.5)


def c_conv_fwd(K, g, small):
    n, cu, pos, start, mx = seg_tables(g, [1] if small else [5, 130, 64])
    return K.conv_silu_fwd(g.bf(n, 64), g.bf(64, 4), start)


def c_conv_bwd(K, g, small):
    n, cu, pos, start, mx = seg_tables(g, [1] if small else [5, 130, 64])
    return K.conv_silu_bwd(g.bf(n, 64), g.bf(n, 64), g.bf(64, 4), start)


def c_quant_fp8(K, g, small):
    r, c = (1, 64) if small else (333, 256)
    q, s = K.quant_fp8_rowwise(g.bf(r, c))
    return q.view(torch.uint8), s


def c_linear_fwd_fp8(K, g, small):
    m, k, n = gemm_dims(small)
    return K.linear_fwd_fp8(g.bf(m, k, scale=0.1), g.bf(k, n, scale=0.1))


def c_linear_fp8(K, g, small):
    m, k, n = gemm_dims(small)
    xq, xs = K.quant_fp8_rowwise(g.bf(m, k, scale=0.1))
    wq, ws = K.quant_fp8_rowwise(g.bf(n, k, scale=0.1))
    return K.linear_fp8(xq, xs, wq, ws)


CASES = {
    "rmsnorm_fwd": c_rmsnorm_fwd, "rmsnorm_apply": c_rmsnorm_apply, "rmsnorm_bwd": c_rmsnorm_bwd,
    "layernorm_fwd": c_layernorm_fwd, "layernorm_apply": c_layernorm_apply, "layernorm_bwd": c_layernorm_bwd,
    "rope_fwd": c_rope("rope_fwd"), "rope_bwd": c_rope("rope_bwd"), "flash_fwd": c_flash_fwd, "flash_bwd": c_flash_bwd,
    "swiglu_fwd_out": c_swiglu_fwd_out, "swiglu_bwd": c_swiglu_bwd, "swiglu_packed_fwd": c_swiglu_packed_fwd,
    "swiglu_packed_bwd": c_swiglu_packed_bwd, "gelu_fwd_out": c_gelu_fwd_out, "gelu_bwd": c_gelu_bwd,
    "ce_loss_fwd_bwd": c_ce_loss, "embed_fwd": c_embed_fwd, "embed_bwd_accum": c_embed_bwd, "adamw_step": c_adamw,
    "adamw_split_step": c_adamw_split, "sgd_step": c_sgd, "linear_fwd_bf16": c_linear_fwd, "linear_dgrad_bf16": c_linear_dgrad,
    "linear_wgrad_bf16": c_linear_wgrad, "bias_grad": c_bias_grad, "add": c_add, "moe_sort": c_moe_sort, "moe_topk_softmax": c_moe_topk_softmax,
    "moe_topk_sigmoid_noaux": c_moe_topk_sigmoid, "moe_router_bwd": c_moe_router_bwd, "moe_dispatch": moe_case(_dispatch),
    "moe_combine": moe_case(_combine), "moe_dispatch_bwd": moe_case(_dispatch_bwd), "moe_scale_rows": moe_case(_scale_rows),
    "moe_rowdot": moe_case(_rowdot), "moe_grouped_mm": moe_case(_grouped_mm), "moe_grouped_wgrad": moe_case(_grouped_wgrad),
    "dsa_index_scores": c_dsa_scores, "dsa_topk_rows": c_dsa_topk, "l2norm_fwd": c_l2norm_fwd, "l2norm_bwd": c_l2norm_bwd,
    "gated_rmsnorm_fwd": c_gated_rmsnorm_fwd, "gated_rmsnorm_bwd": c_gated_rmsnorm_bwd, "conv_silu_fwd": c_conv_fwd,
    "conv_silu_bwd": c_conv_bwd, "quant_fp8_rowwise": c_quant_fp8, "linear_fwd_fp8": c_linear_fwd_fp8, "linear_fp8": c_linear_fp8,
}


def native_ops():
    resolve_kernels(kernel_set="eager")
    return sorted(op for op, impls in registered_ops().items() if any(k.native for k in impls))


def flat(outs):
    if isinstance(outs, torch.Tensor):
        return [outs]
    res = []
    for o in outs:
        if isinstance(o, torch.Tensor):
            res.append(o)
        elif isinstance(o, (tuple, list)):
            res += flat(o)
    return res


def as_bytes(t):
    return t.detach().contiguous().view(torch.uint8).reshape(-1).cpu()


def test_every_native_op_has_a_write_coverage_case():
    assert sorted(CASES) == native_ops()


@pytest.mark.parametrize("op", sorted(CASES))
@pytest.mark.parametrize("small", [False, True], ids=["regular", "degenerate"])
def test_cases_are_valid_calls_on_the_eager_lane(op, small):
    """The table's calls, on CPU tensors through the eager lane: shapes and argument orders are right, outputs exist."""
    K = resolve_kernels(kernel_set="eager")
    outs = flat(CASES[op](K, G("cpu", 1), small))
    assert outs and all(o.numel() > 0 for o in outs)


def poison_free_memory(byte: int):
    """Fill what the caching allocator will hand out next: one large block (split for requests of 1 MiB and more) and a
    batch of small blocks (the small pool serves requests below 1 MiB from 2 MiB segments)."""
    torch.cuda.synchronize()
    big = torch.empty(768 << 20, dtype=torch.uint8, device="cuda")
    big.fill_(byte)
    small = [torch.empty(512 << 10, dtype=torch.uint8, device="cuda") for _ in range(64)]
    for s in small:
        s.fill_(byte)
    torch.cuda.synchronize()
    del big, small


@pytest.mark.gpu
@pytest.mark.parametrize("op", sorted(CASES))
@pytest.mark.parametrize("small", [False, True], ids=["regular", "degenerate"])
def test_native_op_writes_every_output_byte(op, small):
    K = resolve_kernels()
    if op not in K.native_ops():
        pytest.skip(f"{op} is not served by native code on this device")
    runs = []
    for byte in (0x5A, 0xC3):
        poison_free_memory(byte)
        outs = flat(CASES[op](K, G("cuda", 1), small))
        torch.cuda.synchronize()
        runs.append([as_bytes(o) for o in outs])
        del outs
    assert len(runs[0]) == len(runs[1]) > 0
    for i, (a, b) in enumerate(zip(*runs)):
        assert torch.equal(a, b), f"{op}: output {i} differs between two runs over different poison ({int((a != b).sum())} bytes)"
