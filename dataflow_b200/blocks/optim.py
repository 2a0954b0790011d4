"""Optimizer policy as data: learning-rate schedules (pure functions of the 1-indexed
step), per-field optimizer rules with fnmatch overrides, Muon's Newton–Schulz step,
and the fp32 reference update used by tests.  Parity: reference
``src/dataflow_training/blocks/optim.py:62-383`` and ``kernels/muon.py:30-59``.
"""
from __future__ import annotations

import fnmatch
import math
from dataclasses import dataclass, field
from typing import Any, Mapping

OPTIMIZERS = ("adamw", "sgd", "sgdm", "muon", "frozen")
_PLUGIN_OPTIMIZERS: dict[str, Any] = {}


def register_optimizer(name: str, step_fn) -> None:
    _PLUGIN_OPTIMIZERS[name] = step_fn


@dataclass(frozen=True)
class LRSchedule:
    kind: str = "constant"            # constant | cosine | wsd
    peak_lr: float = 3e-4
    min_lr: float = 0.0
    warmup_steps: int = 0
    total_steps: int = 0
    decay_steps: int = 0              # wsd: length of the final decay

    def at(self, step: int) -> float:
        s = max(int(step), 1)
        if self.warmup_steps and s <= self.warmup_steps:
            return self.peak_lr * s / self.warmup_steps
        if self.kind == "constant" or not self.total_steps:
            return self.peak_lr
        if self.kind == "cosine":
            span = max(self.total_steps - self.warmup_steps, 1)
            p = min(max(s - self.warmup_steps, 0) / span, 1.0)
            return self.min_lr + 0.5 * (self.peak_lr - self.min_lr) * (1 + math.cos(math.pi * p))
        if self.kind == "wsd":
            start = self.total_steps - self.decay_steps
            if s <= start:
                return self.peak_lr
            p = min((s - start) / max(self.decay_steps, 1), 1.0)
            return self.peak_lr + (self.min_lr - self.peak_lr) * p
        raise KeyError(self.kind)

    def to_dict(self) -> dict:
        return dict(vars(self))


def lr_at(hyper: Mapping[str, Any], step: int) -> float:
    sch = hyper.get("schedule")
    if sch is None:
        return float(hyper.get("lr", 3e-4))
    if isinstance(sch, LRSchedule):
        return sch.at(step)
    return LRSchedule(**sch).at(step)


@dataclass(frozen=True)
class OptPolicy:
    """Default rule + fnmatch overrides on ``"<layer>/<field>"``; ``layer_overrides`` replaces the
    default for whole layers."""
    default: str = "adamw"
    overrides: tuple[tuple[str, str], ...] = ()
    layer_overrides: Mapping[int, str] = field(default_factory=dict)
    hyper_overrides: tuple[tuple[str, Mapping[str, Any]], ...] = ()

    def rule_for(self, field_name: str, layer=None, kind: str = "matrix") -> str:
        key = f"{layer}/{field_name}"
        for pat, rule in self.overrides:
            if fnmatch.fnmatchcase(key, pat) or fnmatch.fnmatchcase(field_name, pat):
                return rule
        if layer in self.layer_overrides:
            return self.layer_overrides[layer]
        return self.default


@dataclass(frozen=True)
class MuonRecipePolicy(OptPolicy):
    """Hybrid recipe: matrix fields of transformer blocks use Muon, everything else AdamW."""
    default: str = "muon"

    def rule_for(self, field_name: str, layer=None, kind: str = "matrix") -> str:
        r = super().rule_for(field_name, layer, kind)
        if r == "muon" and (kind != "matrix" or layer in (None, "embed", "head")):
            return "adamw"
        return r


def resolve_opt_policy(spec) -> OptPolicy:
    if isinstance(spec, OptPolicy):
        return spec
    if spec in (None, "adamw", "sgd", "sgdm", "frozen"):
        return OptPolicy(spec or "adamw")
    if spec == "muon":
        return MuonRecipePolicy()
    if isinstance(spec, Mapping):
        return OptPolicy(spec.get("default", "adamw"), tuple(map(tuple, spec.get("overrides", ()))),
                         {int(k): v for k, v in spec.get("layer_overrides", {}).items()})
    raise KeyError(spec)


def freeze(policy: OptPolicy | None = None, *, layers=(), fields=(), pairs=(), embed=False, head=False) -> OptPolicy:
    """Compose a policy in which the listed layers / fields / (layer, field) pairs are frozen."""
    base = policy or OptPolicy()
    ov = list(base.overrides)
    ov += [(f, "frozen") for f in fields]
    ov += [(f"{l}/{f}", "frozen") for l, f in pairs]
    lo = dict(base.layer_overrides)
    lo.update({int(l): "frozen" for l in layers})
    if embed:
        ov.append(("embed/*", "frozen"))
    if head:
        ov.append(("head/*", "frozen"))
    return OptPolicy(base.default, tuple(ov), lo, base.hyper_overrides)


NS_COEFFS = (3.4445, -4.775, 2.0315)


def newton_schulz(G, steps: int = 5):
    """Quintic Newton–Schulz orthogonalisation in bf16 (matrix or batch of matrices)."""
    import torch
    a, b, c = NS_COEFFS
    X = G.to(torch.bfloat16)
    transposed = X.shape[-2] > X.shape[-1]
    if transposed:
        X = X.transpose(-1, -2)
    X = X / (X.float().norm(dim=(-2, -1), keepdim=True) + 1e-7).to(X.dtype)
    for _ in range(steps):
        A = X @ X.transpose(-1, -2)
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    return X.transpose(-1, -2) if transposed else X


def muon_field_step(K, f, w, g, o, lr, hyper, step) -> None:
    """Nesterov momentum in storage dtype, NS orthogonalisation, scale 0.2*sqrt(max(r, c))."""
    mu = hyper.get("momentum", 0.95)
    m = o[f"{f.name}.s0"]
    m.copy_((mu * m.float() + g.float()).to(m.dtype))
    upd = g.float() + mu * m.float()
    O = newton_schulz(upd)
    r, c = w.shape[-2], w.shape[-1]
    scale = 0.2 * math.sqrt(max(r, c))
    wd = hyper.get("weight_decay", 0.0)
    w.copy_((w.float() * (1 - lr * wd) - lr * scale * O.float()).to(w.dtype))


def reference_field_step(rule: str, w, g, state: dict, lr: float, hyper: Mapping[str, Any], step: int):
    """fp32 oracle for one field (tests compare kernels and engine runs against this)."""
    import torch
    wd = hyper.get("weight_decay", 0.0)
    if rule == "frozen":
        return w
    if rule == "adamw":
        b1, b2, eps = hyper.get("beta1", 0.9), hyper.get("beta2", 0.95), hyper.get("eps", 1e-8)
        m = state.setdefault("m", torch.zeros_like(w, dtype=torch.float32))
        v = state.setdefault("v", torch.zeros_like(w, dtype=torch.float32))
        gf = g.float()
        m.mul_(b1).add_(gf, alpha=1 - b1)
        v.mul_(b2).addcmul_(gf, gf, value=1 - b2)
        wf = w.float()
        wf = wf - lr * ((m / (1 - b1 ** step)) / ((v / (1 - b2 ** step)).sqrt() + eps) + wd * wf)
        return wf
    if rule == "sgd":
        return w.float() * (1 - lr * wd) - lr * g.float()
    if rule == "sgdm":
        m = state.setdefault("m", torch.zeros_like(w, dtype=torch.float32))
        m.mul_(hyper.get("momentum", 0.9)).add_(g.float())
        return w.float() * (1 - lr * wd) - lr * m
    raise KeyError(rule)
