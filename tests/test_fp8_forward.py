"""fp8 forward projections as a training option (``linear_precision: fp8``): the dense llama block runs its four large
forward GEMMs on e4m3 operands (per-row activation scales, per-output-column weight scales, fp32 accumulation); backward
stays bf16.  On the host backend the oracle lane does the same rounding, so the option is testable without a device."""
import pytest
import torch

from dataflow_b200.models.families import resolve_family
from dataflow_b200.ops import resolve_kernels
from dataflow_b200.run.driver import Trainer, synthetic_rounds
from dataflow_b200.run.recipe import Recipe


def _losses(hyper, steps=6):
    cfg = resolve_family("llama3").presets["tiny"]()
    tr = Trainer("llama3", cfg, budget_gib=None, device=None, hyper={"lr": 3e-3, "weight_decay": 0.1, **hyper}, seed=3)
    out = [tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, 64, 11, s % 2)) for s in range(steps)]
    tr.close()
    return out


def test_fp8_forward_tracks_the_bf16_run():
    base, f8 = _losses({}), _losses({"linear_precision": "fp8"})
    assert base != f8                                           # the option is live
    assert f8[-1] < f8[0] - 1.0                                 # and it trains
    for a, b in zip(base, f8):
        assert abs(a - b) / a < 0.02


def test_fp8_forward_is_the_same_under_recompute():
    """Recomputed context is produced by the same fp8 projections as the forward's, so a plan that recomputes gives the
    same losses as one that saves everything."""
    cfg = resolve_family("llama3").presets["tiny"]()
    hyper = {"lr": 3e-3, "linear_precision": "fp8"}
    out = []
    for lk in (None, {"recompute_levels": {i: 2 for i in range(cfg.n_layers)}}):
        try:
            tr = Trainer("llama3", cfg, budget_gib=None, device=None, hyper=hyper, seed=3, lower_kwargs=lk)
        except TypeError:
            pytest.skip("this lowering takes no explicit recompute levels")
        out.append([tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, 64, 11, s)) for s in range(3)])
        tr.close()
    assert out[0] == out[1]


def test_linear_fwd_fp8_oracle_is_close_to_the_exact_product():
    K = resolve_kernels(kernel_set="eager")
    g = torch.Generator().manual_seed(0)
    x = torch.randn(96, 256, generator=g).bfloat16()
    w = (torch.randn(256, 160, generator=g) * 0.05).bfloat16()
    add = torch.randn(96, 160, generator=g).bfloat16()
    y = K.linear_fwd_fp8(x, w, add=add)
    full = x.float() @ w.float() + add.float()
    assert y.dtype == torch.bfloat16 and float((y.float() - full).norm() / full.norm()) < 0.05
    out = torch.empty(96, 160, dtype=torch.bfloat16)
    assert K.linear_fwd_fp8(x, w, out=out, add=add) is out and torch.equal(out, y)


def test_recipe_carries_the_option():
    assert "linear_precision" not in Recipe().hyper()
    assert Recipe(linear_precision="fp8").hyper()["linear_precision"] == "fp8"
    with pytest.raises(ValueError):
        Recipe(linear_precision="fp4")


def test_reference_form_families_take_the_option_too():
    """dsv32 (autograd lane): fp8 forward for the dense / shared-expert MLPs and the attention output projection, through an
    autograd function whose backward runs on the unquantised operands."""
    from dataflow_b200.testing.family_gate import run_pair
    base = run_pair("dsv32", steps=3)["engine"]
    f8 = run_pair("dsv32", steps=3, overrides={"linear_precision": "fp8"})
    assert f8["engine"] != base and f8["max_loss_rel"] < 1e-3          # the twin runs the same forms, so it quantises too
    for a, b in zip(base, f8["engine"]):
        assert abs(a - b) / a < 0.02
    from dataflow_b200.models import _forms as F
    g = torch.Generator().manual_seed(1)
    x = torch.randn(48, 64, generator=g, requires_grad=True)
    w = (torch.randn(64, 32, generator=g) * 0.1).requires_grad_(True)
    y = F.linear(x, w, "fp8")
    y.sum().backward()
    assert float((y - x @ w).detach().norm() / (x @ w).detach().norm()) < 0.05
    assert torch.allclose(x.grad, torch.ones(48, 32) @ w.t().detach(), atol=1e-5)       # backward: exact products
    assert F.linear(x[:, :60], w[:60], "fp8").shape == (48, 32)                          # odd widths fall back to the plain product
