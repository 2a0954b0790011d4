"""The torch-facing bindings refuse operands they could not safely dereference on a device.

Nothing here launches a kernel: every call fails its operand check first, so the test runs on a
machine without a GPU (the extension itself loads anywhere the CUDA runtime library is present).
"""
import pytest
import torch


@pytest.fixture(scope="module")
def N():
    from dataflow_b200.ops import native
    return native()


def bf(*shape):
    return torch.zeros(*shape, dtype=torch.bfloat16)


def f32(*shape):
    return torch.zeros(*shape, dtype=torch.float32)


def test_host_tensors_are_refused_before_launch(N):
    x, w = bf(4, 64), bf(64)
    cases = [
        lambda: N.gelu_fwd(x, bf(4, 64)),
        lambda: N.gelu_bwd(x, x, bf(4, 64)),
        lambda: N.add_bf16(x, x, bf(4, 64)),
        lambda: N.rmsnorm_fwd(x, w, bf(4, 64), f32(4), 1e-5),
        lambda: N.rmsnorm_apply(x, w, f32(4), bf(4, 64)),
        lambda: N.layernorm_fwd(x, w, w, bf(4, 64), f32(4), f32(4), 1e-5),
        lambda: N.layernorm_apply(x, w, w, f32(4), f32(4), bf(4, 64)),
        lambda: N.layernorm_bwd(x, x, w, f32(4), f32(4), bf(4, 64), None, None, None, False, f32(4 * 2 * 64)),
        lambda: N.adamw_bf16(bf(64), bf(64), bf(64), bf(64), 1e-3, 0.9, 0.95, 1e-8, 0.0, 1, 1.0),
        lambda: N.adamw_master(f32(64), bf(64), bf(64), f32(64), f32(64), 1e-3, 0.9, 0.95, 1e-8, 0.0, 1, 1.0),
        lambda: N.embed_fwd(torch.zeros(4, dtype=torch.int32), bf(16, 64), bf(4, 64), None, None),
        lambda: N.embed_bwd_sorted(torch.zeros(4, dtype=torch.int32), torch.zeros(4, dtype=torch.int32), bf(4, 64), f32(16, 64), False),
        lambda: N.ce_loss_fwd_bwd(bf(4, 64), torch.zeros(4, dtype=torch.int32), f32(4), None, False, 1.0),
    ]
    for i, call in enumerate(cases):
        with pytest.raises(RuntimeError, match="CUDA"):
            call()


def test_messages_name_the_operand(N):
    with pytest.raises(RuntimeError, match=r"\bx must be a CUDA tensor"):
        N.gelu_fwd(bf(8), bf(8))
