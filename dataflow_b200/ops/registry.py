"""Kernel registry: op name → implementations, resolved once per device into a ``KernelSet``.

Each implementation declares a priority, a capability predicate, whether it is
deterministic, and how it gets scratch memory.  Resolution order is: explicit
override (``DATAFLOW_KERNELS=<impl>`` or ``overrides=``) > ``requires(caps)`` >
highest priority.  ``DATAFLOW_KERNELS=eager`` selects the pure-PyTorch reference
lane everywhere (the CPU path and the oracle of every numerics test).
Contract parity: reference ``src/dataflow_training/kernels/registry.py:39-181``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Callable, Mapping


@dataclass(frozen=True)
class Workspace:
    """How an implementation gets scratch: none, from the caller's arena, or internally."""
    kind: str = "none"            # none | arena | internal
    bytes_fn: Callable[..., int] | None = None

    @staticmethod
    def none() -> "Workspace":
        return Workspace("none")

    @staticmethod
    def arena(bytes_fn: Callable[..., int]) -> "Workspace":
        return Workspace("arena", bytes_fn)

    @staticmethod
    def internal() -> "Workspace":
        return Workspace("internal")


@dataclass(frozen=True)
class KernelImpl:
    op: str
    name: str
    fn: Callable[..., Any]
    priority: int = 0
    requires: Callable[[Mapping[str, Any]], bool] | None = None
    deterministic: bool = True
    workspace: Workspace = field(default_factory=Workspace.none)
    allocates: bool = False
    native: bool = False          # hand-written sm_100a kernel (not a library or eager lane)


_REGISTRY: dict[str, list[KernelImpl]] = {}


def register(op: str, impl: str, fn: Callable[..., Any] | None = None, *, priority: int = 0,
             requires: Callable[[Mapping[str, Any]], bool] | None = None, deterministic: bool = True,
             workspace: Workspace | None = None, allocates: bool = False, native: bool = False):
    """Register ``fn`` as implementation ``impl`` of ``op`` (usable as a decorator)."""
    def deco(f):
        lst = _REGISTRY.setdefault(op, [])
        lst[:] = [k for k in lst if k.name != impl]
        lst.append(KernelImpl(op, impl, f, priority, requires, deterministic,
                              workspace or Workspace.none(), allocates, native))
        return f
    return deco(fn) if fn is not None else deco


def registered_ops() -> dict[str, list[KernelImpl]]:
    return {k: list(v) for k, v in _REGISTRY.items()}


@dataclass(frozen=True)
class KernelCtx:
    """Where kernels enqueue: a raw stream handle and (lazily) the torch stream wrapping it."""
    stream_handle: int = 0
    torch_stream: Any = None


def device_caps(device=None) -> dict[str, Any]:
    """Capabilities the ``requires`` predicates look at."""
    caps: dict[str, Any] = {"cuda": False, "cc": (0, 0), "sm100": False, "native_ops": False}
    try:
        import torch
        if torch.cuda.is_available():
            cc = torch.cuda.get_device_capability(device)
            caps.update(cuda=True, cc=cc, sm100=cc[0] == 10, sms=torch.cuda.get_device_properties(device or 0).multi_processor_count)
            from . import native_available
            caps["native_ops"] = native_available() and cc[0] == 10
    except Exception:
        pass
    return caps


class KernelSet:
    """Resolved table; ops are attributes: ``K.rmsnorm_fwd(...)``."""

    def __init__(self, table: dict[str, KernelImpl], caps: Mapping[str, Any]):
        self._table = dict(table)
        self.caps = dict(caps)

    def __getattr__(self, op: str):
        try:
            return self._table[op].fn
        except KeyError:
            raise AttributeError(f"no kernel registered for op {op!r}") from None

    def impl(self, op: str) -> KernelImpl:
        return self._table[op]

    def has(self, op: str) -> bool:
        return op in self._table

    def ops(self) -> list[str]:
        return sorted(self._table)

    def describe(self) -> dict[str, str]:
        return {op: k.name for op, k in sorted(self._table.items())}

    def all_deterministic(self) -> bool:
        return all(k.deterministic for k in self._table.values())

    def native_ops(self) -> list[str]:
        return sorted(op for op, k in self._table.items() if k.native)


def resolve_kernels(caps: Mapping[str, Any] | None = None, overrides: Mapping[str, str] | None = None,
                    kernel_set: str | None = None) -> KernelSet:
    from . import eager  # noqa: F401  (registers the reference lane)
    from . import library  # noqa: F401
    from . import cuda  # noqa: F401
    caps = dict(caps) if caps is not None else device_caps()
    forced = kernel_set if kernel_set is not None else os.environ.get("DATAFLOW_KERNELS", "")
    overrides = dict(overrides or {})
    table: dict[str, KernelImpl] = {}
    for op, impls in _REGISTRY.items():
        usable = [k for k in impls if k.requires is None or k.requires(caps)]
        pick = None
        want = overrides.get(op) or forced
        if want:
            pick = next((k for k in usable if k.name == want), None)
            if pick is None and op in overrides:
                raise KeyError(f"override {want!r} for op {op!r} is not usable on this device")
        if pick is None:
            if not usable:
                continue
            pick = max(usable, key=lambda k: k.priority)
        table[op] = pick
    return KernelSet(table, caps)
