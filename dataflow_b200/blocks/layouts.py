"""Packed byte layouts: named tensor fields at 256-byte aligned offsets inside one
engine object, plus the dtype policy that decides each trainable field's
parameter / gradient / optimizer-state dtypes.

One object per layer (``W_i``), its gradient twin (``dW_i``) and its optimizer
state (``O_i``: optional fp32 master copy, then the optimizer's slots) are all
``PackedLayout``s derived from the same field list, so sizes are byte-exact and
the planner, the executor and the checkpoint agree on them.  Contract parity:
reference ``src/dataflow_training/blocks/layouts.py:30-317`` (256-byte field
alignment, ``ParamDTypes``, fnmatch ``DTypePolicy``); the fp32-master and fp8
policies are additions.
"""
from __future__ import annotations

import fnmatch
import hashlib
from dataclasses import dataclass, field
from typing import Iterable, Mapping, Sequence

from ..core.types import dtype_nbytes

FIELD_ALIGN = 256


def _align(n: int, a: int = FIELD_ALIGN) -> int:
    return (n + a - 1) // a * a


@dataclass(frozen=True)
class Field:
    name: str
    shape: tuple[int, ...]
    dtype: str = "bf16"
    kind: str = "matrix"          # matrix | vector | embedding | scalar  (optimizer policies key on this)
    init: str = "normal"          # normal | ones | zeros | residual (scaled normal) | custom tag

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= int(s)
        return n

    @property
    def nbytes(self) -> int:
        return dtype_nbytes(self.dtype, self.numel)


@dataclass(frozen=True)
class PackedLayout:
    fields: tuple[Field, ...]

    def __post_init__(self):
        names = [f.name for f in self.fields]
        if len(set(names)) != len(names):
            raise ValueError(f"duplicate field names in layout: {names}")

    def offsets(self) -> dict[str, int]:
        off, out = 0, {}
        for f in self.fields:
            out[f.name] = off
            off = _align(off + f.nbytes)
        return out

    @property
    def size_bytes(self) -> int:
        off = 0
        for f in self.fields:
            off = _align(off + f.nbytes)
        return off

    def field(self, name: str) -> Field:
        for f in self.fields:
            if f.name == name:
                return f
        raise KeyError(name)

    def names(self) -> list[str]:
        return [f.name for f in self.fields]

    def views(self, buffer, device: int | None = None, rows: Mapping[str, int] | None = None) -> dict:
        """name → tensor aliasing ``buffer``.  ``rows`` trims the leading dimension of listed
        fields (content < buffer: an under-full round only touches its content rows)."""
        from ..runtime.interop import torch_view
        offs = self.offsets()
        out = {}
        for f in self.fields:
            shape = f.shape
            if rows and f.name in rows:
                shape = (int(rows[f.name]),) + tuple(shape[1:])
            out[f.name] = torch_view(buffer, shape, f.dtype, offs[f.name], device)
        return out

    def digest(self) -> str:
        h = hashlib.sha256()
        for f in self.fields:
            h.update(f"{f.name}:{f.shape}:{f.dtype};".encode())
        return h.hexdigest()[:16]

    def with_dtype(self, dtype_of) -> "PackedLayout":
        return PackedLayout(tuple(Field(f.name, f.shape, dtype_of(f), f.kind, f.init) for f in self.fields))


@dataclass(frozen=True)
class ParamDTypes:
    """Storage dtypes of one trainable field: parameter, gradient, optimizer slots, optional fp32 master."""
    param: str = "bf16"
    grad: str = "bf16"
    opt: str = "bf16"
    master: str | None = None


@dataclass(frozen=True)
class DTypePolicy:
    """Default dtypes plus fnmatch overrides keyed by ``"<layer>/<field>"`` or ``"<field>"``."""
    default: ParamDTypes = ParamDTypes()
    overrides: tuple[tuple[str, ParamDTypes], ...] = ()

    def for_field(self, field_name: str, layer: str | int | None = None) -> ParamDTypes:
        key = f"{layer}/{field_name}" if layer is not None else field_name
        for pat, dt in self.overrides:
            if fnmatch.fnmatchcase(key, pat) or fnmatch.fnmatchcase(field_name, pat):
                return dt
        return self.default

    @staticmethod
    def named(name: str) -> "DTypePolicy":
        if name in ("bf16", "all_bf16"):
            return DTypePolicy(ParamDTypes("bf16", "bf16", "bf16", None))
        if name in ("bf16_master", "fp32_master", "mixed"):
            return DTypePolicy(ParamDTypes("bf16", "bf16", "fp32", "fp32"))
        if name in ("bf16_master_bf16opt",):
            return DTypePolicy(ParamDTypes("bf16", "bf16", "bf16", "fp32"))
        if name in ("bf16_split_master", "split_master"):
            # exact fp32 master whose high half IS the bf16 weight; only the low 16 bits are optimizer state
            return DTypePolicy(ParamDTypes("bf16", "bf16", "bf16", "lo16"))
        if name == "fp32":
            return DTypePolicy(ParamDTypes("fp32", "fp32", "fp32", None))
        if name in ("fp8", "fp8_block"):
            # matrices train through fp8 GEMMs from a bf16 master; everything else stays bf16
            return DTypePolicy(ParamDTypes("bf16", "bf16", "fp32", "fp32"),
                               (("w_router_bias", ParamDTypes("fp32", "fp32", "fp32", None)),
                                ("w_idx_w", ParamDTypes("fp32", "fp32", "fp32", None))))
        raise KeyError(f"unknown dtype policy {name!r}")

    def to_dict(self) -> dict:
        return {"default": vars(self.default).copy(),
                "overrides": [[p, vars(d).copy()] for p, d in self.overrides]}

    @staticmethod
    def from_dict(d) -> "DTypePolicy":
        if isinstance(d, str):
            return DTypePolicy.named(d)
        return DTypePolicy(ParamDTypes(**d["default"]),
                           tuple((p, ParamDTypes(**v)) for p, v in d.get("overrides", ())))


# number of optimizer slots per field for each optimizer rule
OPT_SLOTS = {"adamw": 2, "sgd": 0, "sgdm": 1, "muon": 1, "frozen": 0}


def weight_layout(fields: Sequence[Field], policy: DTypePolicy, layer=None) -> PackedLayout:
    return PackedLayout(tuple(Field(f.name, f.shape, policy.for_field(f.name, layer).param, f.kind, f.init) for f in fields))


def grad_layout(fields: Sequence[Field], policy: DTypePolicy, layer=None, frozen: Iterable[str] = ()) -> PackedLayout:
    fz = set(frozen)
    return PackedLayout(tuple(Field(f.name, f.shape, policy.for_field(f.name, layer).grad, f.kind, "zeros")
                              for f in fields if f.name not in fz))


def opt_state_layout(fields: Sequence[Field], policy: DTypePolicy, layer=None,
                     rule_of=lambda f: "adamw") -> PackedLayout:
    """Per field: [``<f>.master`` fp32 | ``<f>.mlo`` int16 low half of a split master] then ``<f>.s0`` … one per
    optimizer slot."""
    out: list[Field] = []
    for f in fields:
        dt = policy.for_field(f.name, layer)
        rule = rule_of(f)
        if rule == "frozen":
            continue
        if dt.master == "lo16":
            out.append(Field(f"{f.name}.mlo", f.shape, "int16", f.kind, "zeros"))
        elif dt.master:
            out.append(Field(f"{f.name}.master", f.shape, dt.master, f.kind, "copy"))
        for s in range(OPT_SLOTS[rule]):
            out.append(Field(f"{f.name}.s{s}", f.shape, dt.opt, f.kind, "zeros"))
    return PackedLayout(tuple(out))


def sliced_layout(layout: PackedLayout, world: int, rank: int) -> tuple[int, int]:
    """Equal flat byte slices of a packed object (ZeRO): returns (offset, length) of ``rank``'s slice,
    cut on a 256-byte boundary; the last rank takes the tail."""
    total = layout.size_bytes
    per = _align((total + world - 1) // world)
    lo = min(per * rank, total)
    hi = min(per * (rank + 1), total) if rank < world - 1 else total
    return lo, hi - lo
