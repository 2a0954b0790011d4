"""Families that share the llama-style block (RMSNorm, GQA + RoPE attention, SwiGLU or mixture-of-experts MLP):
one registration helper over ``models.llama3``'s lowering, executables and twin.  A variant is a config:
``qk_norm`` (qwen3), ``n_experts`` / ``top_k`` / ``d_ff_expert`` / ``routing_mode`` (olmoe, qwen3moe)."""
from __future__ import annotations

import dataclasses

from .families import ModelFamily, register_family
from .llama3.blocks import build_llama3_resolver
from .llama3.model import (ShapedLlama3Config, derive_dims, family_layouts, flops_per_token, initial_values, lower_llama3)


def register_llama_like(name: str, presets: dict, **fixed):
    """``fixed``: config fields every preset of the family carries (e.g. ``qk_norm=True``)."""
    def make(kw):
        return lambda: ShapedLlama3Config(**{**kw, **fixed, "family": name})

    def _twin(cfg):
        from .twins.llama3 import Llama3Twin
        return Llama3Twin(cfg)

    def _bridge(cfg, views_of):
        from .twins.llama3 import state_dict_from_engine
        return state_dict_from_engine(cfg, views_of)

    return register_family(ModelFamily(
        name=name, config_type=ShapedLlama3Config, derive_dims=derive_dims, lower=lower_llama3,
        initial_values=initial_values, build_resolver=build_llama3_resolver,
        family_layouts=lambda dims, policy=None, optimizer="adamw": family_layouts(dims, policy, optimizer),
        presets={k: make(v) for k, v in presets.items()}, twin=_twin, bridge=_bridge, block_kinds=("block",),
        flops_per_token=flops_per_token))
