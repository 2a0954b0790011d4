"""Audit battery of the kernel registry: every op has the eager oracle, every native implementation declares its
metadata, every native op is exercised by a GPU numerics test somewhere in the suite, and the ops no other test
touches are compared with the oracle here."""
import glob
import os
import re

import pytest
import torch

from dataflow_b200.ops import registered_ops, resolve_kernels

HERE = os.path.dirname(os.path.abspath(__file__))


def all_ops():
    resolve_kernels(kernel_set="eager")          # imports every lane
    return registered_ops()


def test_every_op_has_the_eager_oracle_and_sane_metadata():
    for op, impls in all_ops().items():
        names = [k.name for k in impls]
        assert "eager" in names, f"{op} has no eager oracle"
        assert len(set(names)) == len(names)
        for k in impls:
            assert k.workspace is not None and callable(k.fn)
            if k.name == "eager":
                assert not k.native
            if k.native:
                assert k.name == "sm100" and k.requires is not None, f"{op}: native code must gate on the device"


def test_eager_kernel_set_resolves_every_op_and_is_deterministic():
    ks = resolve_kernels(kernel_set="eager")
    assert set(ks.ops()) == set(all_ops())
    assert ks.all_deterministic() and ks.native_ops() == []


def test_every_native_op_is_named_by_a_gpu_test():
    gpu_tests = ""
    for p in glob.glob(os.path.join(HERE, "test_*.py")):
        text = open(p).read()
        if "pytest.mark.gpu" in text:
            gpu_tests += text
    missing = [op for op, impls in all_ops().items() if any(k.native for k in impls) and not re.search(rf"\b{op}\b", gpu_tests)]
    assert missing == []


def _pair(op):
    impls = {k.name: k.fn for k in all_ops()[op]}
    return impls["sm100"], impls["eager"]


@pytest.mark.gpu
def test_layernorm_apply_matches_oracle():
    native, oracle = _pair("layernorm_apply")
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(300, 768, device="cuda", generator=g).bfloat16()
    w, b = torch.randn(768, device="cuda", generator=g).bfloat16(), torch.randn(768, device="cuda", generator=g).bfloat16()
    mean, var = x.float().mean(-1), x.float().var(-1, unbiased=False)
    rstd = (var + 1e-5).rsqrt()
    ref = oracle(x.cpu(), w.cpu(), b.cpu(), mean.cpu(), rstd.cpu()).float()
    got = native(x, w, b, mean, rstd).float().cpu()
    assert torch.allclose(got, ref, atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
def test_swiglu_fwd_out_and_swiglu_bwd_match_oracle():
    fwd, fwd_ref = _pair("swiglu_fwd_out")
    bwd, bwd_ref = _pair("swiglu_bwd")
    g = torch.Generator(device="cuda").manual_seed(1)
    h13 = torch.randn(257, 2 * 384, device="cuda", generator=g).bfloat16()
    x1, x3 = h13[:, :384], h13[:, 384:]                      # strided halves of the packed projection
    ds = torch.randn(257, 384, device="cuda", generator=g).bfloat16()
    assert torch.allclose(fwd(x1, x3).float().cpu(), fwd_ref(x1.cpu(), x3.cpu()).float(), atol=2e-2, rtol=2e-2)
    d1, d3 = bwd(ds, x1, x3)
    r1, r3 = bwd_ref(ds.cpu(), x1.cpu(), x3.cpu())
    assert torch.allclose(d1.float().cpu(), r1.float(), atol=3e-2, rtol=3e-2)
    assert torch.allclose(d3.float().cpu(), r3.float(), atol=3e-2, rtol=3e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("momentum", [0.0, 0.9])
def test_sgd_step_matches_oracle(momentum):
    """bf16 storage for weights, gradients and momentum; one rounding per stored value, as the oracle does."""
    native, oracle = _pair("sgd_step")
    g = torch.Generator(device="cuda").manual_seed(2)
    w = torch.randn(10007, device="cuda", generator=g).bfloat16()
    grad = torch.randn(10007, device="cuda", generator=g).bfloat16()
    m = torch.zeros(10007, device="cuda", dtype=torch.bfloat16) if momentum else None
    w_ref, m_ref = w.cpu().clone(), (m.cpu().clone() if m is not None else None)
    for _ in range(3):
        native(w, grad, m, lr=0.05, momentum=momentum, wd=0.01)
        oracle(w_ref, grad.cpu(), m_ref, lr=0.05, momentum=momentum, wd=0.01)
    # fused multiply-adds on the device may round the last bf16 bit differently
    assert torch.allclose(w.float().cpu(), w_ref.float(), atol=2e-2, rtol=1e-2)
    if m is not None:
        assert torch.allclose(m.float().cpu(), m_ref.float(), atol=2e-2, rtol=1e-2)


@pytest.mark.gpu
def test_l2norm_fwd_and_l2norm_bwd_match_oracle():
    fwd, fwd_ref = _pair("l2norm_fwd")
    bwd, bwd_ref = _pair("l2norm_bwd")
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(513, 4, 128, device="cuda", generator=g).bfloat16()
    dy = torch.randn(513, 4, 128, device="cuda", generator=g).bfloat16()
    y, r = fwd(x)
    y_ref, r_ref = fwd_ref(x.cpu())
    assert torch.allclose(y.float().cpu(), y_ref.float(), atol=1e-2, rtol=1e-2) and torch.allclose(r.cpu(), r_ref, rtol=1e-4)
    assert torch.allclose(bwd(dy, x, r).float().cpu(), bwd_ref(dy.cpu(), x.cpu(), r_ref).float(), atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
def test_gated_rmsnorm_fwd_and_gated_rmsnorm_bwd_match_oracle():
    fwd, fwd_ref = _pair("gated_rmsnorm_fwd")
    bwd, bwd_ref = _pair("gated_rmsnorm_bwd")
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(700, 8, 128, device="cuda", generator=g).bfloat16()
    gate = torch.randn(700, 8, 128, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(128, device="cuda", generator=g)).bfloat16()
    dy = torch.randn(700, 8, 128, device="cuda", generator=g).bfloat16()
    y, r = fwd(x, gate, w)
    y_ref, r_ref = fwd_ref(x.cpu(), gate.cpu(), w.cpu())
    assert torch.allclose(y.float().cpu(), y_ref.float(), atol=3e-2, rtol=3e-2)
    dx, dg, dw = bwd(dy, x, gate, w, r)
    rx, rg, rw = bwd_ref(dy.cpu(), x.cpu(), gate.cpu(), w.cpu(), r_ref)
    for a, b in ((dx, rx), (dg, rg), (dw, rw)):
        assert float((a.float().cpu() - b.float()).norm() / b.float().norm()) < 1e-2


@pytest.mark.gpu
def test_conv_silu_fwd_and_conv_silu_bwd_match_oracle():
    fwd, fwd_ref = _pair("conv_silu_fwd")
    bwd, bwd_ref = _pair("conv_silu_bwd")
    g = torch.Generator(device="cuda").manual_seed(5)
    n, c = 333, 200
    x = torch.randn(n, c, device="cuda", generator=g).bfloat16()
    w = (0.5 * torch.randn(c, 4, device="cuda", generator=g)).bfloat16()
    dy = torch.randn(n, c, device="cuda", generator=g).bfloat16()
    start = torch.tensor([0] * 100 + [100] * 133 + [233] * 100, dtype=torch.int32, device="cuda")
    assert torch.allclose(fwd(x, w, start).float().cpu(), fwd_ref(x.cpu(), w.cpu(), start.cpu()).float(), atol=3e-2, rtol=3e-2)
    dx, dw = bwd(dy, x, w, start)
    rx, rw = bwd_ref(dy.cpu(), x.cpu(), w.cpu(), start.cpu())
    assert float((dx.float().cpu() - rx.float()).norm() / rx.float().norm()) < 1e-2
    assert float((dw.cpu() - rw).norm() / rw.norm()) < 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("groups", [(1, 1), (4, 2)])
def test_moe_topk_sigmoid_noaux_matches_oracle(groups):
    native, oracle = _pair("moe_topk_sigmoid_noaux")
    g = torch.Generator(device="cuda").manual_seed(6)
    logits = torch.randn(1000, 64, device="cuda", generator=g).bfloat16()
    bias = 0.1 * torch.randn(64, device="cuda", generator=g)
    w, ids = native(logits, bias, 6, groups[0], groups[1], 2.5)
    w_ref, ids_ref = oracle(logits.cpu(), bias.cpu(), 6, groups[0], groups[1], 2.5)
    same = (ids.cpu().sort(-1).values == ids_ref.sort(-1).values.to(torch.int32)).all(-1)
    assert same.float().mean() > 0.995                    # ties between nearly equal bf16 scores may break differently
    assert torch.allclose(w.cpu().sum(-1), torch.full((1000,), 2.5), atol=1e-4)
    assert torch.allclose(w.cpu()[same].sort(-1).values, w_ref[same].sort(-1).values, atol=1e-4)


@pytest.mark.gpu
def test_quant_fp8_rowwise_matches_oracle():
    native, oracle = _pair("quant_fp8_rowwise")
    g = torch.Generator(device="cuda").manual_seed(7)
    x = (torch.randn(300, 1024, device="cuda", generator=g) * torch.logspace(-2, 2, 300, device="cuda")[:, None]).bfloat16()
    x[17].zero_()
    q, s = native(x)
    q_ref, s_ref = oracle(x.cpu())
    assert torch.allclose(s.cpu(), s_ref, rtol=1e-6)
    # conversions round to nearest in both lanes; allow the odd tie to land on the neighbouring code
    same = (q.cpu().view(torch.uint8) == q_ref.view(torch.uint8)).float().mean()
    assert same > 0.999
    back = q.float() * s[:, None]
    assert float((back - x.float()).norm() / x.float().norm()) < 0.04


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(512, 768, 1024), (4096, 4096, 4096), (300, 520, 272)])
def test_linear_fp8_matches_oracle(shape):
    """The tcgen05 fp8 GEMM (kind::f8f6f4, fp32 accumulate) with its dequantising epilogue against the same product in fp32."""
    quant, _ = _pair("quant_fp8_rowwise")
    native, oracle = _pair("linear_fp8")
    m, n, k = shape
    g = torch.Generator(device="cuda").manual_seed(8)
    x = torch.randn(m, k, device="cuda", generator=g).bfloat16()
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16()
    resid = torch.randn(m, n, device="cuda", generator=g).bfloat16()
    xq, sx = quant(x)
    wq, sw = quant(w)
    y = native(xq, sx, wq, sw, add=resid)
    y_ref = oracle(xq.cpu(), sx.cpu(), wq.cpu(), sw.cpu(), add=resid.cpu())
    assert float((y.float().cpu() - y_ref.float()).norm() / y_ref.float().norm()) < 5e-3
    # and the quantised product stays close to the bf16 one
    full = x.float() @ w.float().t() + resid.float()
    assert float((y.float() - full).norm() / full.norm()) < 0.06
    from dataflow_b200.ops import native as _n
    assert _n().gemm_last_error() == 0


@pytest.mark.gpu
def test_linear_fwd_fp8_matches_oracle():
    """The composed forward linear (quantise activations per row, the (in, out) weight per output column, fp8 GEMM) against
    the same composition in the oracle, and against the bf16 product."""
    native, oracle = _pair("linear_fwd_fp8")
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(1000, 1024, device="cuda", generator=g).bfloat16()
    w = (torch.randn(1024, 768, device="cuda", generator=g) * 0.03).bfloat16()
    resid = torch.randn(1000, 768, device="cuda", generator=g).bfloat16()
    out = torch.empty(1000, 768, device="cuda", dtype=torch.bfloat16)
    y = native(x, w, out=out, add=resid)
    assert y.data_ptr() == out.data_ptr()
    y_ref = oracle(x.cpu(), w.cpu(), add=resid.cpu())
    assert float((y.float().cpu() - y_ref.float()).norm() / y_ref.float().norm()) < 5e-3
    full = x.float() @ w.float() + resid.float()
    assert float((y.float() - full).norm() / full.norm()) < 0.06
