"""A complete family defined OUTSIDE the package, the way a user's plugin would: importing this module registers it
(``DATAFLOW_PLUGINS=tests.fixtures.external_family.toy_family`` or ``--plugin`` on the tools).  Two kinds of layers:
a token-mixing layer (causal running mean inside each segment, then a linear map) and a gated MLP layer.
Reference role: ``tests/fixtures/external_family/toy_family.py``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from dataflow_b200.blocks.layouts import DTypePolicy, Field
from dataflow_b200.models import _forms as F
from dataflow_b200.models._torch_family import TorchFamilySpec, register_torch_family


@dataclass(frozen=True)
class ToyConfig:
    name: str = "toy"
    n_layers: int = 4
    d_model: int = 64
    d_ff: int = 128
    vocab_size: int = 256
    rms_eps: float = 1e-6
    seq_len: int = 32
    batch: int = 2
    grad_accum_rounds: int = 2
    dtype_policy: Any = "bf16"
    optimizer: str = "adamw"
    optimizer_placement: str = "interleaved"
    head_chunk_tokens: int = 2048
    family: str = "toy"

    def policy(self) -> DTypePolicy:
        return self.dtype_policy if isinstance(self.dtype_policy, DTypePolicy) else DTypePolicy.from_dict(self.dtype_policy)

    @property
    def tokens_per_round(self) -> int:
        return self.seq_len * self.batch


def layer_kinds(c):
    return ["mix" if i % 2 == 0 else "mlp" for i in range(c.n_layers)]


def kind_fields(c, kind):
    d = c.d_model
    if kind == "mix":
        return (Field("norm", (d,), "bf16", "vector", "ones"), Field("w_mix", (d, d), "bf16", "matrix", "residual"))
    return (Field("norm", (d,), "bf16", "vector", "ones"), Field("w13", (d, 2 * c.d_ff)), Field("w2", (c.d_ff, d), "bf16", "matrix", "residual"))


def block_fn(c, kind, x, w, seg, layer):
    h = F.rmsnorm(x, w["norm"], c.rms_eps)
    if kind == "mlp":
        return x + F.swiglu_mlp(h, w["w13"], w["w2"]), None
    n = x.shape[0]
    mask = F.segment_causal_mask(seg, n, x.device).to(h.dtype)
    mean = (mask @ h) / mask.sum(-1, keepdim=True)
    return x + mean @ w["w_mix"], None


def kind_flops(c, kind, tokens):
    d = c.d_model
    return (2.0 * tokens * d * d, 2.0 * tokens * c.seq_len * d) if kind == "mix" else (2.0 * tokens * 3 * d * c.d_ff, 0.0)


SPEC = TorchFamilySpec("toy", ToyConfig, {"tiny": lambda: ToyConfig()}, layer_kinds, kind_fields, block_fn, kind_flops)
FAMILY = register_torch_family(SPEC)
