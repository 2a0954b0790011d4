"""Scalar vocabulary of the Program IR: locations, roles, dtypes, tensor metadata.

Parity: ``src/dataflow/core/types.py:12-86`` of the reference (same names, same
dtype bit table, dense-stride convention).  stdlib only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Literal, Sequence

Location = Literal["fast", "backing"]
LOCATIONS: tuple[str, ...] = ("fast", "backing")

Role = str
ROLES: tuple[str, ...] = (
    "parameter", "gradient", "optimizer_state", "activation",
    "input", "output", "temp", "other",
)

# bits per element; sub-byte types are packed
DTYPE_BITS: dict[str, int] = {
    "fp64": 64, "fp32": 32, "tf32": 32, "fp16": 16, "bf16": 16,
    "fp8_e4m3": 8, "fp8_e5m2": 8, "fp4": 4,
    "int64": 64, "int32": 32, "int16": 16, "int8": 8, "uint8": 8, "bool": 8,
}


def dtype_nbytes(dtype: str, count: int) -> int:
    """Bytes needed to store ``count`` elements of ``dtype`` (packed, rounded up)."""
    try:
        bits = DTYPE_BITS[dtype]
    except KeyError:
        raise ValueError(f"unknown dtype {dtype!r}") from None
    return (bits * int(count) + 7) // 8


@dataclass(frozen=True)
class TensorMeta:
    """Optional dense-tensor view of an object's bytes.

    ``strides`` are in elements; ``None`` means row-major contiguous.
    """

    dtype: str
    shape: tuple[int, ...]
    strides: tuple[int, ...] | None = None

    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= int(s)
        return n

    def dense_strides(self) -> tuple[int, ...]:
        out: list[int] = []
        acc = 1
        for s in reversed(self.shape):
            out.append(acc)
            acc *= int(s)
        return tuple(reversed(out))

    def is_dense(self) -> bool:
        return self.strides is None or tuple(self.strides) == self.dense_strides()

    def nbytes(self) -> int:
        return dtype_nbytes(self.dtype, self.numel())


def as_shape(shape: Sequence[int]) -> tuple[int, ...]:
    return tuple(int(s) for s in shape)
