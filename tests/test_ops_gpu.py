"""Numerics of every hand-written sm_100a kernel against the plain PyTorch fp32 reference of the
same op (the ``eager`` lane), plus the write-coverage check: running an op twice with different
poison in its outputs must give identical bytes."""
import pytest
import torch

from dataflow_b200.ops import eager, resolve_kernels

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def K():
    k = resolve_kernels()
    assert k.caps["sm100"], "these tests expect a Blackwell GPU"
    assert len(k.native_ops()) >= 20, f"native kernels not selected: {k.describe()}"
    return k


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("rows,cols", [(7, 64), (300, 4096), (1000, 768), (33, 200), (700, 2048), (310, 8192), (5000, 4096)])
def test_rmsnorm_fwd_bwd(K, rows, cols):
    torch.manual_seed(0)
    x, w, dy, add = bf(rows, cols), bf(cols) + 1, bf(rows, cols), bf(rows, cols)
    y, rstd = K.rmsnorm_fwd(x, w, 1e-5)
    yr, rr = eager.rmsnorm_fwd(x.float(), w.float(), 1e-5)
    assert rel(y, yr) < 5e-3 and rel(rstd, rr) < 1e-5
    assert rel(K.rmsnorm_apply(x, w, rstd), yr) < 5e-3
    if cols % 8:
        return
    for acc in (False, True):
        dw = bf(cols)
        dw_ref = dw.float().clone()
        dx = K.rmsnorm_bwd(dy, x, w, rstd, dx_add=add, dw=dw, accumulate=acc)
        dxr = eager.rmsnorm_bwd(dy.float(), x.float(), w.float(), rr, dx_add=add.float(), dw=dw_ref, accumulate=acc)
        assert rel(dx, dxr) < 5e-3 and rel(dw, dw_ref) < 1e-2


@pytest.mark.parametrize("rows,cols", [(64, 768), (257, 1024)])
def test_layernorm_fwd_bwd(K, rows, cols):
    torch.manual_seed(1)
    x, w, b, dy = bf(rows, cols) + 0.5, bf(cols) + 1, bf(cols), bf(rows, cols)
    y, mean, rstd = K.layernorm_fwd(x, w, b, 1e-5)
    yr, mr, rr = eager.layernorm_fwd(x.float(), w.float(), b.float(), 1e-5)
    assert rel(y, yr) < 5e-3 and rel(mean, mr) < 1e-4 and rel(rstd, rr) < 1e-4
    dw, db = torch.zeros(cols, device=DEV, dtype=torch.bfloat16), torch.zeros(cols, device=DEV, dtype=torch.bfloat16)
    dwr, dbr = torch.zeros(cols, device=DEV), torch.zeros(cols, device=DEV)
    dx = K.layernorm_bwd(dy, x, w, mean, rstd, dw=dw, db=db)
    dxr = eager.layernorm_bwd(dy.float(), x.float(), w.float(), mr, rr, dw=dwr, db=dbr)
    assert rel(dx, dxr) < 5e-3 and rel(dw, dwr) < 1e-2 and rel(db, dbr) < 1e-2


def test_rope_strided_and_inverse(K):
    torch.manual_seed(2)
    t, hq, hkv, hd = 300, 8, 2, 128
    qkv = bf(t, (hq + 2 * hkv) * hd)
    pos = torch.arange(t, device=DEV, dtype=torch.int32) % 97
    ref = qkv.float().clone()
    q = qkv[:, :hq * hd].unflatten(1, (hq, hd))
    K.rope_fwd(q, pos, 500000.0)
    eager.rope_fwd(ref[:, :hq * hd].unflatten(1, (hq, hd)), pos, 500000.0)
    assert rel(qkv, ref) < 5e-3
    assert torch.equal(qkv[:, hq * hd:].float(), ref[:, hq * hd:])        # untouched columns
    k = qkv[:, hq * hd:(hq + hkv) * hd].unflatten(1, (hkv, hd))             # two heads: one head per thread
    K.rope_fwd(k, pos, 500000.0)
    eager.rope_fwd(ref[:, hq * hd:(hq + hkv) * hd].unflatten(1, (hkv, hd)), pos, 500000.0)
    assert rel(qkv, ref) < 5e-3
    assert torch.equal(qkv[:, (hq + hkv) * hd:].float(), ref[:, (hq + hkv) * hd:])
    z = bf(t, 3, 20)                                                          # pairs too short for 16-byte accesses
    zr = z.float().clone()
    K.rope_fwd(z, pos, 10000.0)
    eager.rope_fwd(zr, pos, 10000.0)
    assert rel(z, zr) < 5e-3
    orig = bf(t, hq, hd)
    x = orig.clone()
    K.rope_fwd(x, pos, 10000.0)
    K.rope_bwd(x, pos, 10000.0)
    assert rel(x, orig) < 1e-2
    # partial rotation at a column base (MLA-style decoupled rope)
    y = bf(t, 4, 192)
    yr = y.float().clone()
    K.rope_fwd(y, pos, 10000.0, rot_dim=64, col_base=128)
    eager.rope_fwd(yr, pos, 10000.0, rot_dim=64, col_base=128)
    assert rel(y, yr) < 5e-3


def test_swiglu_gelu_add(K):
    torch.manual_seed(3)
    rows, F = 513, 1024
    h13, ds = bf(rows, 2 * F), bf(rows, F)
    s = K.swiglu_packed_fwd(h13)
    assert rel(s, eager.swiglu_packed_fwd(h13)) < 2e-3
    d = K.swiglu_packed_bwd(ds, h13)
    assert rel(d, eager.swiglu_packed_bwd(ds.float(), h13.float())) < 5e-3
    d2, s2 = K.swiglu_packed_bwd(ds, h13, with_s=True)
    assert torch.equal(d2, d) and torch.equal(s2, s)                          # the product rides along, same bytes as the forward
    big = bf(2048, 2 * 8192)                                                  # more vectors than one pass of the grid holds
    assert rel(K.swiglu_packed_fwd(big), eager.swiglu_packed_fwd(big)) < 2e-3
    x, dy = bf(rows, F), bf(rows, F)
    assert rel(K.gelu_fwd_out(x), eager.gelu_fwd_out(x.float())) < 5e-3
    assert rel(K.gelu_bwd(dy, x), eager.gelu_bwd(dy.float(), x.float())) < 5e-3
    assert rel(K.add(x, dy), x.float() + dy.float()) < 5e-3


@pytest.mark.parametrize("rows,vocab", [(64, 1000), (300, 50304), (17, 128256)])
def test_ce_loss(K, rows, vocab):
    torch.manual_seed(4)
    logits = bf(rows, vocab, scale=2.0)
    tgt = torch.randint(0, vocab, (rows,), device=DEV, dtype=torch.int32)
    tgt[::5] = -1
    ref_logits = logits.float().clone()
    loss = K.ce_loss_fwd_bwd(logits, tgt, 1000.0)
    loss_ref = eager.ce_loss_fwd_bwd(ref_logits, tgt, 1000.0)
    assert abs(loss.item() - loss_ref.item()) < 1e-3 * abs(loss_ref.item()) + 1e-6
    assert rel(logits, ref_logits) < 1e-2
    assert torch.all(logits[::5] == 0)


def test_embed_fwd_bwd_deterministic(K):
    torch.manual_seed(5)
    vocab, d, t = 1000, 256, 4096
    table, dy = bf(vocab, d), bf(t, d)
    tok = torch.randint(0, 50, (t,), device=DEV, dtype=torch.int32)       # heavy collisions
    assert torch.equal(K.embed_fwd(tok, table), table[tok.long()])
    g1, g2 = torch.full((vocab, d), 7.0, device=DEV, dtype=torch.bfloat16), torch.full((vocab, d), -3.0, device=DEV, dtype=torch.bfloat16)
    K.embed_bwd_accum(tok, dy, g1, accumulate=False)
    K.embed_bwd_accum(tok, dy, g2, accumulate=False)
    assert torch.equal(g1, g2)                                           # create ignores previous bytes; order is fixed
    ref = torch.zeros(vocab, d, device=DEV)
    eager.embed_bwd_accum(tok, dy.float(), ref)
    assert rel(g1, ref) < 5e-3
    K.embed_bwd_accum(tok, dy, g1, accumulate=True)
    assert rel(g1, 2 * ref) < 1e-2


def test_adamw_variants(K):
    torch.manual_seed(6)
    n = 100_003
    hp = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1)
    w, g = bf(n), bf(n)
    m, v = torch.zeros(n, device=DEV, dtype=torch.bfloat16), torch.zeros(n, device=DEV, dtype=torch.bfloat16)
    wr, mr, vr = w.clone(), m.clone(), v.clone()
    for step in (1, 2, 3):
        K.adamw_step(w, g, m, v, step=step, **hp)
        eager.adamw_step(wr, g, mr, vr, step=step, **hp)
    assert rel(w, wr) < 2e-3 and rel(m, mr) < 5e-3
    master = torch.randn(n, device=DEV)
    w2 = master.to(torch.bfloat16)
    m32, v32 = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    mref, wref2, m2, v2 = master.clone(), w2.clone(), m32.clone(), v32.clone()
    for step in (1, 2):
        K.adamw_step(w2, g, m32, v32, step=step, master=master, **hp)
        eager.adamw_step(wref2, g, m2, v2, step=step, master=mref, **hp)
    assert rel(master, mref) < 1e-5 and torch.equal(w2, master.to(torch.bfloat16))


@pytest.mark.parametrize("M,N,K_", [(128, 256, 64), (200, 264, 136), (1024, 768, 512), (4096, 1024, 2048)])
def test_linear_triple_matches_fp32(K, M, N, K_):
    torch.manual_seed(7)
    x, w, dy, add = bf(M, K_), bf(K_, N, scale=0.05), bf(M, N), bf(M, N)
    y = K.linear_fwd_bf16(x, w, add=add)
    assert rel(y, x.float() @ w.float() + add.float()) < 5e-3
    dx = K.linear_dgrad_bf16(dy, w)
    assert rel(dx, dy.float() @ w.float().t()) < 5e-3
    dw = torch.full((K_, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.linear_wgrad_bf16(x, dy, dw, accumulate=False)
    ref = x.float().t() @ dy.float()
    assert rel(dw, ref) < 5e-3
    K.linear_wgrad_bf16(x, dy, dw, accumulate=True)
    assert rel(dw, 2 * ref) < 1e-2
    dw32 = torch.zeros(K_, N, device=DEV)
    K.linear_wgrad_bf16(x, dy, dw32, accumulate=False)
    assert rel(dw32, ref) < 1e-5
    from dataflow_b200.ops import native
    assert native().gemm_last_error() == 0


def test_bias_grad_and_write_coverage(K):
    torch.manual_seed(8)
    dy = bf(1000, 768)
    for poison in (5.0, -9.0):
        db = torch.full((768,), poison, device=DEV, dtype=torch.bfloat16)
        K.bias_grad(dy, db)
        assert rel(db, dy.float().sum(0)) < 5e-3


@pytest.mark.gpu
@pytest.mark.parametrize("shape", ["uniform", "ragged"])
def test_attention_library_lane_matches_the_reference(shape):
    """Uniform rounds take the cuDNN fused attention, ragged ones the varlen flash kernels; both must reproduce the
    fp32 reference (output, log-sum-exp, and all three gradients), GQA included, on strided views of a packed qkv."""
    import torch
    from dataflow_b200.ops import registered_ops, resolve_kernels
    resolve_kernels()
    impls = {op: {k.name: k.fn for k in registered_ops()[op]} for op in ("flash_fwd", "flash_bwd")}
    hq, hkv, d = 8, 2, 128
    bounds = [0, 256, 512, 768, 1024] if shape == "uniform" else [0, 192, 448, 1024]
    t = bounds[-1]
    g = torch.Generator(device="cuda").manual_seed(5)
    qkv = (torch.randn(t, (hq + 2 * hkv) * d, device="cuda", generator=g) * 0.5).bfloat16()
    q = qkv[:, :hq * d].unflatten(1, (hq, d))
    k = qkv[:, hq * d:(hq + hkv) * d].unflatten(1, (hkv, d))
    v = qkv[:, (hq + hkv) * d:].unflatten(1, (hkv, d))
    cu = torch.tensor(bounds, dtype=torch.int32, device="cuda")
    mx = max(b - a for a, b in zip(bounds[:-1], bounds[1:]))
    o, lse = impls["flash_fwd"]["baseline"](q, k, v, cu, mx)
    o_ref, lse_ref = impls["flash_fwd"]["eager"](q.cpu(), k.cpu(), v.cpu(), torch.tensor(bounds), mx)
    assert torch.allclose(o.float().cpu(), o_ref.float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(lse.cpu(), lse_ref, atol=2e-3, rtol=2e-3)
    do = (torch.randn(t, hq, d, device="cuda", generator=g) * 0.5).bfloat16()
    dq, dk, dv = impls["flash_bwd"]["baseline"](do, q, k, v, o, lse, cu, mx)
    rq, rk, rv = impls["flash_bwd"]["eager"](do.cpu(), q.cpu(), k.cpu(), v.cpu(), o_ref, lse_ref, torch.tensor(bounds), mx)
    for a, b in ((dq, rq), (dk, rk), (dv, rv)):
        assert float((a.float().cpu() - b.float()).norm() / b.float().norm()) < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("shape", ["uniform", "ragged", "long", "short"])
def test_flash_fwd_tcgen05_kernel_matches_the_reference(shape):
    """The hand-written tcgen05 forward (TMA loads, S and P V in tensor memory, online softmax in registers) against the fp32
    reference: output and log-sum-exp, GQA, strided views of a packed qkv, sequences that end inside a tile."""
    import torch
    from dataflow_b200.ops import native, registered_ops, resolve_kernels
    resolve_kernels()
    impls = {k.name: k.fn for k in registered_ops()["flash_fwd"]}
    hq, hkv, d = 8, 2, 128
    bounds = {"uniform": [0, 256, 512, 768, 1024], "ragged": [0, 100, 457, 460, 1024], "long": [0, 2048], "short": [0, 1, 64, 65, 193]}[shape]
    t = bounds[-1]
    g = torch.Generator(device="cuda").manual_seed(9)
    qkv = (torch.randn(t, (hq + 2 * hkv) * d, device="cuda", generator=g) * 0.7).bfloat16()
    q = qkv[:, :hq * d].unflatten(1, (hq, d))
    k = qkv[:, hq * d:(hq + hkv) * d].unflatten(1, (hkv, d))
    v = qkv[:, (hq + hkv) * d:].unflatten(1, (hkv, d))
    cu = torch.tensor(bounds, dtype=torch.int32, device="cuda")
    mx = max(b - a for a, b in zip(bounds[:-1], bounds[1:]))
    from dataflow_b200.ops.cuda import flash_fwd_tcgen05
    o, lse = flash_fwd_tcgen05(q, k, v, cu, mx)
    torch.cuda.synchronize()
    assert native().gemm_last_error() == 0
    if shape == "ragged":                       # the default lane sends ragged rounds to the same kernel
        o2, lse2 = impls["sm100"](q, k, v, cu, mx)
        assert torch.equal(o2, o) and torch.equal(lse2, lse)
    o_ref, lse_ref = impls["eager"](q.cpu(), k.cpu(), v.cpu(), torch.tensor(bounds), mx)
    assert torch.allclose(lse.cpu(), lse_ref, atol=3e-3, rtol=3e-3)
    assert float((o.float().cpu() - o_ref.float()).norm() / o_ref.float().norm()) < 1e-2
    assert torch.allclose(o.float().cpu(), o_ref.float(), atol=3e-2, rtol=3e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", ["uniform", "ragged", "long", "short"])
def test_flash_bwd_tcgen05_kernels_match_the_reference(shape):
    """The hand-written tcgen05 backward (dK / dV kernel with keys as accumulator rows, dQ kernel, both recomputing the
    scores in tensor memory) against the fp32 reference: dq, dk, dv, GQA summed over the group, strided views of packed
    qkv / dqkv buffers, sequences that end inside a tile; the result is bitwise repeatable and covers every output byte."""
    import torch
    from dataflow_b200.ops import native, registered_ops, resolve_kernels
    from dataflow_b200.ops.cuda import flash_bwd_tcgen05, flash_fwd_tcgen05
    resolve_kernels()
    impls = {op: {k.name: k.fn for k in registered_ops()[op]} for op in ("flash_fwd", "flash_bwd")}
    hq, hkv, d = 8, 2, 128
    bounds = {"uniform": [0, 256, 512, 768, 1024], "ragged": [0, 100, 457, 460, 1024], "long": [0, 2048], "short": [0, 1, 64, 65, 193]}[shape]
    t = bounds[-1]
    g = torch.Generator(device="cuda").manual_seed(11)
    qkv = (torch.randn(t, (hq + 2 * hkv) * d, device="cuda", generator=g) * 0.7).bfloat16()
    q = qkv[:, :hq * d].unflatten(1, (hq, d))
    k = qkv[:, hq * d:(hq + hkv) * d].unflatten(1, (hkv, d))
    v = qkv[:, (hq + hkv) * d:].unflatten(1, (hkv, d))
    cu = torch.tensor(bounds, dtype=torch.int32, device="cuda")
    mx = max(b - a for a, b in zip(bounds[:-1], bounds[1:]))
    o, lse = flash_fwd_tcgen05(q, k, v, cu, mx)
    do = (torch.randn(t, hq, d, device="cuda", generator=g) * 0.5).bfloat16()
    outs = []
    for poison in (3.0, -7.0):
        dqkv = torch.full((t, (hq + 2 * hkv) * d), poison, device="cuda", dtype=torch.bfloat16)
        dq = dqkv[:, :hq * d].unflatten(1, (hq, d))
        dk = dqkv[:, hq * d:(hq + hkv) * d].unflatten(1, (hkv, d))
        dv = dqkv[:, (hq + hkv) * d:].unflatten(1, (hkv, d))
        flash_bwd_tcgen05(do, q, k, v, o, lse, cu, mx, dq=dq, dk=dk, dv=dv)
        torch.cuda.synchronize()
        assert native().gemm_last_error() == 0
        outs.append(dqkv)
    assert torch.equal(outs[0], outs[1])                    # every byte written, the same way, whatever was there before
    o_ref, lse_ref = impls["flash_fwd"]["eager"](q.cpu(), k.cpu(), v.cpu(), torch.tensor(bounds), mx)
    rq, rk, rv = impls["flash_bwd"]["eager"](do.cpu(), q.cpu(), k.cpu(), v.cpu(), o_ref, lse_ref, torch.tensor(bounds), mx)
    for name, a, b in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        err = float((a.float().cpu() - b.float()).norm() / b.float().norm())
        assert err < 2e-2, (name, err)
    d2 = impls["flash_bwd"]["sm100"](do, q, k, v, o, lse, cu, mx)       # the default lane is this kernel
    assert torch.equal(d2[0], dq) and torch.equal(d2[1], dk) and torch.equal(d2[2], dv)


@pytest.mark.parametrize("n,H,D,bounds", [(300, 4, 64, [0, 300]), (1000, 8, 128, [0, 137, 700, 1000]), (2500, 64, 128, [0, 2500]),
                                           (130, 3, 128, [0, 5, 130])])
def test_dsa_index_scores_on_tcgen05_match_the_fp32_form(K, n, H, D, bounds):
    """Indexer scores (ReLU-weighted sum over heads fused behind the tensor-core product, visibility mask applied) against
    the eager fp32 form of the same bf16 inputs; blocks of query rows; ragged sequences; written twice over different poison."""
    torch.manual_seed(n)
    q, k = bf(n, H, D, scale=D ** -0.25), bf(n, D, scale=D ** -0.25)
    wgt = torch.randn(n, H, device=DEV)
    seg_start = torch.cat([torch.full((b - a,), a, dtype=torch.int32) for a, b in zip(bounds[:-1], bounds[1:])]).to(DEV)
    for q0, q1 in ((0, n), (128, min(n, 640)), (n - 70, n)):
        if q0 >= q1:
            continue
        got = K.dsa_index_scores(q, k, wgt, seg_start, q0, q1, 0)
        want = eager.dsa_index_scores(q, k, wgt, seg_start, q0, q1, 0)
        fin = torch.isfinite(want)
        assert torch.equal(torch.isfinite(got), fin)
        assert torch.equal(got[~fin], want[~fin])               # -inf exactly where the query does not see the key
        assert rel(got[fin], want[fin]) < 2e-3
    torch.cuda.synchronize()


@pytest.mark.parametrize("rows,cols,k", [(5, 40, 12), (64, 3000, 256), (33, 16384, 2048), (9, 100, 100), (4, 50, 80)])
def test_dsa_topk_rows_is_exact_and_deterministic(K, rows, cols, k):
    """The selection kernel against a stable sort: the k largest of every row, ties to the smaller index, ascending indices,
    -1 for rows with fewer finite entries; ReLU-like inputs with many exact ties; two runs over different poison agree."""
    torch.manual_seed(cols)
    s = torch.relu(torch.randn(rows, cols, device=DEV)) * (torch.rand(rows, cols, device=DEV) > 0.3)      # many zeros
    s[:, int(cols * 0.8):] = float("-inf")
    s[0] = float("-inf")
    if rows > 2:
        s[2, : cols // 2] = 1.5                                                                              # one long tie
    want = eager.dsa_topk_rows(s, k, 7)
    outs = []
    for poison in (-3, 12345):
        sel = torch.full((rows, k), poison, dtype=torch.int32, device=DEV)
        from dataflow_b200.ops import native
        native().dsa_topk_rows(s, rows, cols, 7, k, sel)
        outs.append(sel)
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(outs[0].cpu(), want.cpu())
    assert torch.equal(K.dsa_topk_rows(s, k, 7), outs[0])
