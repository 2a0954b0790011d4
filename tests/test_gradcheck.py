"""Per-tensor gradient checks of the engine lowerings against autograd through the twins (`testing/gradcheck.py`)."""
import pytest

from dataflow_b200.ops import resolve_kernels
from dataflow_b200.testing.gradcheck import CheckReport, check_block_backward, check_model_step, rel_l2


@pytest.mark.parametrize("family", ["llama3", "gpt2", "qwen3", "qwen35"])
def test_dense_families_match_autograd_per_tensor(family):
    rep = check_model_step(family)
    assert rep, rep.summary()
    assert len(rep.grad_rel_l2) >= 10 and rep.loss_rel < 1e-4


@pytest.mark.parametrize("family", ["olmoe", "dsv3"])
def test_moe_families_match_autograd_within_the_routing_band(family):
    rep = check_model_step(family, tol=0.25)
    assert rep, rep.summary()
    dense = {k: v for k, v in rep.grad_rel_l2.items() if any(s in k for s in ("w_qkv", "wq_a", "wkv_a", "wte"))}
    assert dense and max(dense.values()) < 5e-2


@pytest.mark.parametrize("family,over", [("dsv3", {"top_k": 8, "n_group": 1, "topk_group": 1}), ("olmoe", {"top_k": 8})])
def test_moe_gradients_are_dense_tight_once_routing_cannot_flip(family, over):
    """With every expert selected there is no discrete choice left for rounding to flip: the dispatch, grouped GEMMs, combine
    and router backward then agree with autograd as closely as the dense blocks do."""
    rep = check_model_step(family, overrides=over)
    assert rep, rep.summary()
    assert max(rep.grad_rel_l2.values()) < 2e-2


def test_block_backward_reports_one_layers_fields_and_ragged_rounds_pass():
    rep = check_block_backward("llama3", shape="ragged")
    assert rep, rep.summary()
    assert set(k.split(".")[1] for k in rep.grad_rel_l2) == {"0"} and "layers.0.w13" in rep.grad_rel_l2
    mixed = check_block_backward("qwen35", kind_layer=3)           # the fourth layer of the hybrid is the gated-attention kind
    assert mixed and all(k.startswith("layers.3.") for k in mixed.grad_rel_l2)


def test_a_wrong_backward_is_caught():
    good = resolve_kernels(kernel_set="eager")

    class Wrong:
        def __getattr__(self, name):
            return getattr(good, name)

        def swiglu_packed_bwd(self, ds, h13, *a, **k):
            out = good.swiglu_packed_bwd(ds, h13, *a, **k)
            (out[0] if isinstance(out, tuple) else out).mul_(0.5)      # half the gradient through the gate
            return out

    rep = check_model_step("llama3", kernels=Wrong())
    assert not rep
    bad = rep.failures()
    assert "layers.0.w13" in bad and bad["layers.0.w13"] > 0.3
    assert "layers.1.w2" not in bad                                    # tensors downstream of the fault are still right


def test_report_arithmetic():
    import torch
    assert rel_l2(torch.ones(4), torch.ones(4)) == 0.0
    r = CheckReport("x", 1.0, 1.0, {"a": 0.5, "b": 0.5}, {"a": 1.0, "b": 0.0})
    assert set(r.failures()) == {"a"} and not r                        # zero-gradient tensors have no direction to compare
    assert "worst" in r.summary()
