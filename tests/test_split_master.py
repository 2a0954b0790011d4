"""Split fp32 master (bf16 weight = high half, int16 plane = low half): exactness of the split and the
AdamW step built on it, on the eager lane (CPU) and the sm_100a kernel (GPU)."""
import pytest
import torch

from dataflow_b200.ops import eager


def test_split_is_exact_roundtrip():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1 << 16, generator=g) * torch.logspace(-6, 3, 1 << 16)
    x[:4] = torch.tensor([0.0, -0.0, 1.0, -1.0])
    # ties: low half exactly 0x8000
    t = torch.tensor([0x3F808000, 0xBF808000, 0x3F7F8000], dtype=torch.int64).to(torch.int32).view(torch.float32)
    x = torch.cat([x, t])
    w, lo = eager.split_master_cut(x)
    back = eager.split_master_join(w, lo)
    assert torch.equal(back.view(torch.int32), x.view(torch.int32))
    # the working weight is within half a bf16 ulp of the master
    assert ((w.float() - x).abs() <= (x.abs() * 2 ** -8 + 1e-45)).all()


def _ref_steps(w0, grads, lr, wd, steps):
    master = w0.float().clone()
    m = torch.zeros_like(master, dtype=torch.bfloat16)
    v = torch.zeros_like(master, dtype=torch.bfloat16)
    for s in range(1, steps + 1):
        gf = grads[s - 1].float()
        m = (0.9 * m.float() + 0.1 * gf).bfloat16()
        v = (0.95 * v.float() + 0.05 * gf * gf).bfloat16()
        mh = m.float() / (1 - 0.9 ** s)
        vh = v.float() / (1 - 0.95 ** s)
        master = master - lr * (mh / (vh.sqrt() + 1e-8) + wd * master)
    return master


def test_split_adamw_tracks_fp32_master():
    g = torch.Generator().manual_seed(1)
    n = 4099
    w = torch.randn(n, generator=g).bfloat16()
    lo = torch.zeros(n, dtype=torch.int16)
    m = torch.zeros(n, dtype=torch.bfloat16)
    v = torch.zeros(n, dtype=torch.bfloat16)
    grads = [(torch.randn(n, generator=g) * 0.1).bfloat16() for _ in range(5)]
    w0 = w.clone()
    for s, gr in enumerate(grads, 1):
        eager.adamw_split_step(w, lo, gr, m, v, 1e-3, 0.9, 0.95, 1e-8, 0.1, s)
    ref = _ref_steps(w0, grads, 1e-3, 0.1, 5)
    got = eager.split_master_join(w, lo)
    assert torch.allclose(got, ref, rtol=1e-6, atol=1e-7)
    # a plain bf16 weight would have lost these updates: the master differs from the bf16 weight
    assert (got != w.float()).any()


@pytest.mark.gpu
def test_split_adamw_kernel_matches_eager():
    from dataflow_b200.ops import native
    g = torch.Generator().manual_seed(2)
    for n in (8, 4099, 1 << 20):
        w = torch.randn(n, generator=g).bfloat16()
        lo = torch.randint(-32768, 32767, (n,), generator=g, dtype=torch.int32).to(torch.int16)
        m = (torch.randn(n, generator=g) * 0.01).bfloat16()
        v = (torch.rand(n, generator=g) * 1e-4).bfloat16()
        gr = (torch.randn(n, generator=g) * 0.1).bfloat16()
        dw, dlo, dm, dv, dg = (t.cuda() for t in (w, lo, m, v, gr))
        native().adamw_split(dw, dlo, dg, dm, dv, 3e-4, 0.9, 0.95, 1e-8, 0.1, 3, 1.0)
        eager.adamw_split_step(w, lo, gr, m, v, 3e-4, 0.9, 0.95, 1e-8, 0.1, 3)
        torch.cuda.synchronize()
        got = eager.split_master_join(dw.cpu(), dlo.cpu())
        ref = eager.split_master_join(w, lo)
        # (1 - beta) is formed in fp32 on the device and in double on the host: now and then a moment lands on the
        # neighbouring bf16 value, which moves that element's update by a fraction of a percent
        diff = (got - ref).abs()
        assert float((diff <= 1e-6 + 2e-6 * ref.abs()).float().mean()) > 0.995, n
        assert torch.allclose(got, ref, rtol=1e-4, atol=1e-4), n
        assert torch.allclose(dm.cpu().float(), m.float(), rtol=1e-2, atol=1e-6)
        assert torch.allclose(dv.cpu().float(), v.float(), rtol=1e-2, atol=1e-9)
