"""gpt2 family registration and presets."""
from __future__ import annotations

from ..families import ModelFamily, register_family
from .blocks import build_gpt2_resolver
from .model import (Gpt2Dims, ShapedGpt2Config, derive_dims, family_layouts, flops_per_token, initial_values, lower_gpt2)


def _p(**kw):
    return lambda: ShapedGpt2Config(**kw)


PRESETS = {
    "tiny": _p(name="tiny", n_layers=2, d_model=128, n_heads=4, vocab_size=512, max_positions=128, seq_len=64, batch=2,
               grad_accum_rounds=2),
    # untied, vocab padded to a multiple of 64, bf16: the reference's default training preset
    "gpt2_124m": _p(name="gpt2_124m", n_layers=12, d_model=768, n_heads=12, vocab_size=50304, max_positions=1024,
                    seq_len=1024, batch=8, grad_accum_rounds=8),
    # tied embeddings, exact vocab, fp32 everything, seq 1024, batch 2, 2 accumulation rounds: the CPU plumbing configuration
    "gpt2_124m_fp32": _p(name="gpt2_124m_fp32", n_layers=12, d_model=768, n_heads=12, vocab_size=50257, max_positions=1024,
                         seq_len=1024, batch=2, grad_accum_rounds=2, tied_embeddings=True, dtype_policy="fp32",
                         act_dtype="fp32", head_chunk_tokens=512),
}


def _twin(cfg):
    from ..twins.gpt2 import Gpt2Twin
    return Gpt2Twin(cfg)


def _bridge(cfg, views_of):
    from ..twins.gpt2 import state_dict_from_engine
    return state_dict_from_engine(cfg, views_of)


FAMILY = register_family(ModelFamily(
    name="gpt2", config_type=ShapedGpt2Config, derive_dims=derive_dims, lower=lower_gpt2,
    initial_values=initial_values, build_resolver=build_gpt2_resolver,
    family_layouts=lambda dims, policy=None, optimizer="adamw": family_layouts(dims, policy, optimizer),
    presets=PRESETS, twin=_twin, bridge=_bridge, block_kinds=("block",), flops_per_token=flops_per_token))
