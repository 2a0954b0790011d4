"""Training recipe: the optimizer hyper-parameters of a run as data.  ``Recipe.hyper()`` is the dict the
executables read (``blocks.optim.lr_at`` evaluates the schedule as a pure function of the 1-indexed step).
Defaults follow the reference's recipe (betas 0.9 / 0.95, weight decay 0.1, cosine to min_lr, no clipping):
``src/dataflow_training/run/recipe.py:24`` and ``run/schedule.py:22``.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any

from ..blocks.optim import LRSchedule


@dataclass(frozen=True)
class Recipe:
    peak_lr: float = 3e-4
    min_lr: float = 3e-5
    warmup_steps: int = 0
    total_steps: int = 0
    schedule: str = "cosine"            # constant | cosine | wsd
    decay_steps: int = 0
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    optimizer: str = "adamw"
    muon_lr: float | None = None
    momentum: float = 0.95
    linear_precision: str = "bf16"      # bf16 | fp8: operand precision of the dense forward projections (llama-like families)

    def __post_init__(self):
        if self.linear_precision not in ("bf16", "fp8"):
            raise ValueError(f"linear_precision must be bf16 or fp8, not {self.linear_precision!r}")

    def lr_schedule(self) -> LRSchedule:
        return LRSchedule(self.schedule, self.peak_lr, self.min_lr, self.warmup_steps, self.total_steps, self.decay_steps)

    def lr(self, step: int) -> float:
        return self.lr_schedule().at(step)

    def hyper(self) -> dict[str, Any]:
        h = {"optimizer": self.optimizer, "lr": self.peak_lr, "schedule": self.lr_schedule().to_dict(), "beta1": self.beta1,
             "beta2": self.beta2, "eps": self.eps, "weight_decay": self.weight_decay, "momentum": self.momentum}
        if self.muon_lr is not None:
            h["muon_lr"] = self.muon_lr
        if self.linear_precision != "bf16":
            h["linear_precision"] = self.linear_precision
        return h

    def to_dict(self) -> dict:
        return asdict(self)


CosineSchedule = LRSchedule     # the schedule object itself (kind="cosine")
