"""Parameter initialisation as data: which rule fills which field.

A rule is a NAME plus arguments, resolved through a registry of fill callables (names travel in configs and over the
service's wire; callables do not).  A policy is a default rule, ordered ``fnmatch`` overrides on field names, and layer
routing (a layer listed in ``layer_overrides`` is answered entirely by its sub-policy).  Every fill draws from the ONE
seeded CPU generator in field order, in fp32, and is cast to the field's storage dtype: the same seed gives the same bytes
on every machine and at every world size.

The default policy is "what the layout says": a field's own ``init`` tag (``normal`` std 0.02, ``ones``, ``zeros``,
``residual`` = normal scaled by 1 / sqrt(2 L)).  A run that names a policy (``hyper["init_policy"]``, wire form below)
overrides that per field:

    {"default": {"rule": "normal", "args": {"std": 0.01}},
     "overrides": [["*_norm", {"rule": "constant", "args": {"value": 1.0}}],
                   ["w2", {"rule": "scaled_normal", "args": {"std": 0.02, "divide_by": 8.0}}]],
     "layer_overrides": [[[0, 1], {"default": {"rule": "normal", "args": {"std": 0.05}}}]]}

Role parity: reference ``src/dataflow_training/model_families/init_policy.py:1-140``.
"""
from __future__ import annotations

import contextlib
import contextvars
from dataclasses import dataclass, field
from fnmatch import fnmatchcase
from typing import Any, Callable

INIT_RULES: dict[str, Callable[..., Callable]] = {}


def register_init_rule(name: str, build: Callable[..., Callable]) -> None:
    """``build(**args)`` returns ``fill(n, gen) -> flat fp32 tensor of n elements``."""
    INIT_RULES[name] = build


def _normal(std: float = 0.02, mean: float = 0.0):
    def fill(n, gen):
        import torch
        t = torch.empty(n, dtype=torch.float32).normal_(0.0, float(std), generator=gen)
        return t + float(mean) if mean else t
    return fill


def _constant(value: float = 0.0):
    def fill(n, gen):
        import torch
        return torch.full((n,), float(value), dtype=torch.float32)
    return fill


def _scaled_normal(std: float = 0.02, divide_by: float = 1.0):
    return _normal(float(std) / float(divide_by))


def _uniform(low: float = -0.02, high: float = 0.02):
    def fill(n, gen):
        import torch
        return torch.empty(n, dtype=torch.float32).uniform_(float(low), float(high), generator=gen)
    return fill


for _name, _build in (("normal", _normal), ("constant", _constant), ("scaled_normal", _scaled_normal), ("uniform", _uniform)):
    register_init_rule(_name, _build)


@dataclass(frozen=True)
class InitRule:
    name: str
    args: dict = field(default_factory=dict)

    def build(self) -> Callable:
        if self.name not in INIT_RULES:
            raise KeyError(f"unknown init rule {self.name!r} (registered: {sorted(INIT_RULES)})")
        return INIT_RULES[self.name](**self.args)

    def to_dict(self) -> dict:
        return {"rule": self.name, "args": dict(self.args)}


@dataclass(frozen=True)
class InitPolicy:
    """``default`` None = the field's own tag decides (the layouts' built-in behaviour)."""
    default: InitRule | None = None
    overrides: tuple = ()                    # ((fnmatch pattern on the field name, InitRule), ...): first match wins
    layer_overrides: tuple = ()              # (((layer, ...), InitPolicy), ...)

    def rule(self, name: str, layer: int | None = None) -> InitRule | None:
        if layer is not None:
            for layers, sub in self.layer_overrides:
                if layer in layers:
                    return sub.rule(name, None)
        for pattern, r in self.overrides:
            if fnmatchcase(name, pattern):
                return r
        return self.default

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"overrides": [[p, r.to_dict()] for p, r in self.overrides],
                             "layer_overrides": [[list(ls), sub.to_dict()] for ls, sub in self.layer_overrides]}
        if self.default is not None:
            d["default"] = self.default.to_dict()
        return d


DEFAULT_INIT_POLICY = InitPolicy()


def build_init_policy(spec: dict | InitPolicy | None) -> InitPolicy:
    """Wire / config form -> policy; ``None`` -> the default (byte-identical to the layouts' tags)."""
    if spec is None:
        return DEFAULT_INIT_POLICY
    if isinstance(spec, InitPolicy):
        return spec

    def rule(d):
        return InitRule(d["rule"], dict(d.get("args") or {}))
    return InitPolicy(default=rule(spec["default"]) if spec.get("default") else None,
                      overrides=tuple((p, rule(r)) for p, r in spec.get("overrides", ())),
                      layer_overrides=tuple((tuple(int(i) for i in ls), build_init_policy(sub)) for ls, sub in spec.get("layer_overrides", ())))


_ACTIVE: contextvars.ContextVar = contextvars.ContextVar("dataflow_init_policy", default=(DEFAULT_INIT_POLICY, None))


@contextlib.contextmanager
def init_scope(policy: InitPolicy | dict | None, layer: int | None = None):
    """The policy (and, inside a layer's object, the layer index) that ``fill_by_policy`` consults."""
    tok = _ACTIVE.set((build_init_policy(policy), layer))
    try:
        yield
    finally:
        _ACTIVE.reset(tok)


@contextlib.contextmanager
def layer_scope(layer: int | None):
    pol, _ = _ACTIVE.get()
    tok = _ACTIVE.set((pol, layer))
    try:
        yield
    finally:
        _ACTIVE.reset(tok)


def set_init_layer(object_id: str) -> None:
    """Called by a family's init loop in front of every weight object: ``W_7`` -> layer 7, ``W_embed`` / ``W_head`` -> none."""
    pol, _ = _ACTIVE.get()
    tail = object_id.split("_", 1)[-1]
    _ACTIVE.set((pol, int(tail) if tail.isdigit() else None))


def fill_by_policy(t, field_name: str, gen) -> bool:
    """Fill ``t`` by the active policy's rule for this field; False when the policy leaves the field to its own tag."""
    pol, layer = _ACTIVE.get()
    r = pol.rule(field_name, layer)
    if r is None:
        return False
    fill = r.build()
    flat = t.reshape(-1)
    step = 1 << 24
    for lo in range(0, flat.numel(), step):
        n = min(step, flat.numel() - lo)
        flat[lo:lo + n].copy_(fill(n, gen))
    return True
