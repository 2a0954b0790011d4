"""qwen35moe family: the qwen35 hybrid stack (gated delta-rule layers, every fourth layer gated softmax attention) with a
mixture-of-experts MLP — softmax top-k routing, a load-balance term, and one shared expert whose output passes a
sigmoid gate.  Kinds ``linattnmoe`` and ``gattnmoe``.
Family parity: reference ``src/dataflow_training/model_families/qwen35moe/blocks.py:50-139``.
"""
from __future__ import annotations

from ..qwen35 import Qwen35Config, block_fn, kind_fields, kind_flops, layer_kinds
from .._torch_family import TorchFamilySpec, register_torch_family

MOE = dict(n_experts=8, top_k=2, d_ff_expert=64, shared_expert=True, aux_coef=0.01, family="qwen35moe")
PRESETS = {
    "tiny": dict(name="tiny", **MOE),
    "qwen35moe_20l": dict(name="qwen35moe_20l", n_layers=20, d_model=2048, lin_k_heads=16, lin_v_heads=32, lin_dk=128, lin_dv=128, n_heads=16,
                          n_kv_heads=2, head_dim=256, vocab_size=151936, rope_theta=1e7, seq_len=4096, batch=1, grad_accum_rounds=8,
                          **{**MOE, "n_experts": 128, "top_k": 8, "d_ff_expert": 512}),
    "qwen35moe_35b": dict(name="qwen35moe_35b", n_layers=48, d_model=2048, lin_k_heads=16, lin_v_heads=32, lin_dk=128, lin_dv=128, n_heads=16,
                          n_kv_heads=2, head_dim=256, vocab_size=151936, rope_theta=1e7, seq_len=4096, batch=1, grad_accum_rounds=16,
                          dtype_policy="bf16_split_master", **{**MOE, "n_experts": 256, "top_k": 8, "d_ff_expert": 512}),
}

SPEC = TorchFamilySpec("qwen35moe", Qwen35Config, {k: (lambda kw=v: Qwen35Config(**kw)) for k, v in PRESETS.items()}, layer_kinds, kind_fields,
                       block_fn, kind_flops, ep_fields=("w13_experts", "w2_experts"))
FAMILY = register_torch_family(SPEC)
