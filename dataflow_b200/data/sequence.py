"""The units the data plane moves: one ``Sequence`` (a document / record / window with its targets), one
``PackedRound`` (the fixed-size int32 buffers of a grad-accumulation round plus its segment bounds) and one
``PackedStep`` (all rounds of an optimizer step plus the cursor that resumes the source right after it).
Contract parity: reference ``src/dataflow_training/data/sequence.py:18-91``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

import numpy as np

IGNORE_INDEX = -1


@dataclass
class Sequence:
    tokens: np.ndarray                       # (n,) int32
    targets: np.ndarray                      # (n,) int32, IGNORE_INDEX = no loss at this position
    extras: dict[str, np.ndarray] = field(default_factory=dict)

    def __post_init__(self):
        self.tokens = np.ascontiguousarray(self.tokens, dtype=np.int32)
        self.targets = np.ascontiguousarray(self.targets, dtype=np.int32)
        if self.tokens.ndim != 1 or self.tokens.shape != self.targets.shape:
            raise ValueError(f"tokens {self.tokens.shape} and targets {self.targets.shape} must be equal 1-D arrays")
        for k, v in self.extras.items():
            if len(v) != len(self.tokens):
                raise ValueError(f"extra {k!r} has {len(v)} entries for {len(self.tokens)} tokens")

    def __len__(self) -> int:
        return int(self.tokens.shape[0])

    @property
    def real_targets(self) -> int:
        return int((self.targets >= 0).sum())

    def slice(self, a: int, b: int) -> "Sequence":
        return Sequence(self.tokens[a:b], self.targets[a:b], {k: v[a:b] for k, v in self.extras.items()})

    @staticmethod
    def from_document(ids, eot: int | None) -> "Sequence":
        """Next-token shift inside one document; the last position targets ``eot`` (masked when there is none)."""
        ids = np.asarray(ids, dtype=np.int32)
        tg = np.empty_like(ids)
        tg[:-1] = ids[1:]
        tg[-1] = IGNORE_INDEX if eot is None else eot
        return Sequence(ids, tg)


@dataclass
class PackedRound:
    tokens: np.ndarray                       # (tokens_per_round,) int32, tail beyond ``content`` is filler
    targets: np.ndarray                      # (tokens_per_round,) int32, tail is IGNORE_INDEX
    bounds: list[int]                        # [0, b1, ..., content]: segment edges inside the round
    content: int                             # tokens that are real data

    @property
    def valid_rows(self) -> int:
        return int((self.targets[:self.content] >= 0).sum())

    @property
    def fill(self) -> float:
        return self.content / float(len(self.tokens)) if len(self.tokens) else 0.0


@dataclass
class PackedStep:
    rounds: list[PackedRound]
    cursor_after: Mapping[str, Any]          # JSON-able: resumes the source right after this step
    index: int = 0

    @property
    def valid_rows(self) -> int:
        return sum(r.valid_rows for r in self.rounds)

    @property
    def content_tokens(self) -> int:
        return sum(r.content for r in self.rounds)

    @property
    def fill(self) -> float:
        cap = sum(len(r.tokens) for r in self.rounds)
        return self.content_tokens / float(cap) if cap else 0.0

    def seq_lens(self, execute_padding: bool = False) -> dict[int, list[int]]:
        """``run_args["seq_lens"]``: per round, the bounds ending at the content edge (or, with
        ``execute_padding``, one more masked segment out to the buffer size)."""
        out = {}
        for r, rd in enumerate(self.rounds):
            b = list(rd.bounds)
            if execute_padding and rd.content < len(rd.tokens):
                b.append(len(rd.tokens))
            out[r] = b
        return out

    def digest(self) -> str:
        import hashlib
        h = hashlib.sha256()
        for rd in self.rounds:
            h.update(rd.tokens[:rd.content].tobytes())
            h.update(rd.targets[:rd.content].tobytes())
            h.update(np.asarray(rd.bounds, dtype=np.int64).tobytes())
        return h.hexdigest()[:16]
