"""dsv32 family (DeepSeek-V3.2 architecture): dsv3 plus sparse attention — a lightning indexer (a few small heads, one
shared key, ReLU scores) ranks the visible keys of every query, attention runs over the ``index_topk`` best, and the
indexer is trained by a KL term towards the attention distribution (gradient injected in the block backward; the
attention side is a constant target).  Kinds ``dsadense`` / ``dsamoe``.
Dense warm-up (``dsa_warmup=True``, presets ``*_warmup``): attention stays dense, the indexer learns the full-prefix
attention distribution through the same KL term and the optimizer updates nothing but the indexer's fields (``wi_*``).
Family parity: reference ``src/dataflow_training/model_families/dsv32/{blocks.py,model.py}`` (warm-up variants :584-658).
"""
from __future__ import annotations

import dataclasses

from ..dsv3 import EP_FIELDS, Dsv3Config, block_fn as _block_fn, kind_fields as _kind_fields, kind_flops
from .._torch_family import TorchFamilySpec, register_torch_family


def layer_kinds(c: Dsv3Config):
    return ["dsadense" if i < c.n_dense else "dsamoe" for i in range(c.n_layers)]


BASE = dict(index_heads=2, index_dim=16, index_topk=32, index_kl_coef=0.1, family="dsv32")
PRESETS = {
    "tiny": dict(name="tiny", **BASE),
    "tiny_warmup": dict(name="tiny_warmup", dsa_warmup=True, **BASE),
    "dsv32_mini": dict(name="dsv32_mini", n_layers=6, n_dense=1, d_model=512, n_heads=8, q_lora=192, kv_lora=128, d_nope=64, d_rope=32, d_v=64,
                       d_ff=1408, n_experts=16, top_k=4, d_ff_expert=256, n_group=4, topk_group=2, vocab_size=32000, seq_len=1024, batch=4,
                       grad_accum_rounds=4, **{**BASE, "index_heads": 4, "index_dim": 32, "index_topk": 256}),
    "dsv32_671b": dict(name="dsv32_671b", n_layers=61, n_dense=3, d_model=7168, n_heads=128, q_lora=1536, kv_lora=512, d_nope=128, d_rope=64,
                       d_v=128, d_ff=18432, n_experts=256, top_k=8, d_ff_expert=2048, n_group=8, topk_group=4, routed_scaling=2.5,
                       vocab_size=129280, seq_len=4096, batch=1, grad_accum_rounds=16, dtype_policy="bf16_split_master",
                       **{**BASE, "index_heads": 64, "index_dim": 128, "index_topk": 2048}),
    # the 12-layer cut used as a multi-GPU benchmark configuration: 3 dense layers, 256 routed experts (top-8) + 1 shared,
    # indexer top-2048 at 16k tokens per sequence, experts split over the ranks (``ep`` set by ``--parallel ep``)
    # long-context exercise of the sparse lane on one GPU: full-size indexer (64 heads of 128, top-2048) and latent widths, a
    # narrow model around them
    "dsv32_long16k": dict(name="dsv32_long16k", n_layers=4, n_dense=1, d_model=2048, n_heads=32, q_lora=768, kv_lora=512, d_nope=128, d_rope=64,
                          d_v=128, d_ff=8192, n_experts=16, top_k=4, d_ff_expert=1024, n_group=4, topk_group=2, routed_scaling=2.5,
                          vocab_size=32000, seq_len=16384, batch=1, grad_accum_rounds=1, dtype_policy="bf16",
                          **{**BASE, "index_heads": 64, "index_dim": 128, "index_topk": 2048}),
    "dsv32_12l": dict(name="dsv32_12l", n_layers=12, n_dense=3, d_model=7168, n_heads=128, q_lora=1536, kv_lora=512, d_nope=128, d_rope=64,
                      d_v=128, d_ff=18432, n_experts=256, top_k=8, d_ff_expert=2048, n_group=8, topk_group=4, routed_scaling=2.5,
                      vocab_size=129280, seq_len=16384, batch=1, grad_accum_rounds=8, dtype_policy="bf16_split_master",
                      linear_precision="fp8", **{**BASE, "index_heads": 64, "index_dim": 128, "index_topk": 2048}),
}

SPEC = TorchFamilySpec("dsv32", Dsv3Config, {k: (lambda kw=v: Dsv3Config(**kw)) for k, v in PRESETS.items()}, layer_kinds, _kind_fields,
                       _block_fn, kind_flops, ep_fields=EP_FIELDS)
FAMILY = register_torch_family(SPEC)
