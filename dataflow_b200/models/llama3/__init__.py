"""llama3 family registration and presets (tiny, the l3 ladder, 8B, 70B)."""
from __future__ import annotations

from ..families import ModelFamily, register_family
from .blocks import build_llama3_resolver
from .model import (Llama3Dims, ShapedLlama3Config, derive_dims, family_layouts, flops_per_token,
                    initial_values, lower_llama3)


def _p(**kw):
    return lambda: ShapedLlama3Config(**kw)


PRESETS = {
    "tiny": _p(name="tiny", n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, d_ff=512, vocab_size=1024,
               seq_len=128, batch=2, grad_accum_rounds=2),
    "l3_125m": _p(name="l3_125m", n_layers=12, d_model=768, n_heads=12, n_kv_heads=4, head_dim=64, d_ff=2048,
                  vocab_size=50304, seq_len=2048, batch=4, grad_accum_rounds=8),
    "l3_350m": _p(name="l3_350m", n_layers=24, d_model=1024, n_heads=16, n_kv_heads=4, head_dim=64, d_ff=2816,
                  vocab_size=50304, seq_len=2048, batch=4, grad_accum_rounds=8),
    "l3_760m": _p(name="l3_760m", n_layers=24, d_model=1536, n_heads=12, n_kv_heads=4, head_dim=128, d_ff=4096,
                  vocab_size=50304, seq_len=2048, batch=4, grad_accum_rounds=8),
    "l3_1b": _p(name="l3_1b", n_layers=16, d_model=2048, n_heads=16, n_kv_heads=8, head_dim=128, d_ff=8192,
                vocab_size=50304, seq_len=2048, batch=4, grad_accum_rounds=8),
    "llama3_8b": _p(name="llama3_8b", n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, d_ff=14336,
                    vocab_size=128256, seq_len=4096, batch=4, grad_accum_rounds=8, dtype_policy="bf16_master"),
    "llama3_70b": _p(name="llama3_70b", n_layers=80, d_model=8192, n_heads=64, n_kv_heads=8, head_dim=128, d_ff=28672,
                     vocab_size=128256, seq_len=8192, batch=2, grad_accum_rounds=8, dtype_policy="bf16_master"),
}


def _layouts(dims, policy=None, optimizer="adamw"):
    return family_layouts(dims, policy, optimizer)


def _twin(cfg):
    from ..twins.llama3 import Llama3Twin
    return Llama3Twin(cfg)


def _bridge(cfg, views_of):
    from ..twins.llama3 import state_dict_from_engine
    return state_dict_from_engine(cfg, views_of)


FAMILY = register_family(ModelFamily(
    name="llama3", config_type=ShapedLlama3Config, derive_dims=derive_dims, lower=lower_llama3,
    initial_values=initial_values, build_resolver=build_llama3_resolver, family_layouts=_layouts,
    presets=PRESETS, twin=_twin, bridge=_bridge, block_kinds=("block",), flops_per_token=flops_per_token))
