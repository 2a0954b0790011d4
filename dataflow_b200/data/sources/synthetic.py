"""Seeded random sequences (benchmarks and tests without data).  Sequence ``i`` is a pure function of
``(seed, i)``: uniform ids, length drawn around ``mean_len`` (fixed when ``jitter == 0``), next-token targets
with the last position masked.  Parity: reference ``src/dataflow_training/data/sources/synthetic.py``.
"""
from __future__ import annotations

import numpy as np

from ..sequence import Sequence
from . import DataSource


class SyntheticSource(DataSource):
    scheme = "synthetic"

    def __init__(self, vocab: int = 50257, mean_len: int = 512, seed: int = 0, jitter: float = 0.5, **kw):
        super().__init__(**kw)
        self.vocab, self.mean_len, self.seed, self.jitter = int(vocab), int(mean_len), int(seed), float(jitter)

    def start_cursor(self) -> dict:
        return {"index": 0}

    def raw(self, cursor):
        i = int(cursor.get("index", 0))
        while True:
            g = np.random.default_rng([self.seed, i])
            lo = max(2, int(self.mean_len * (1 - self.jitter)))
            hi = max(lo + 1, int(self.mean_len * (1 + self.jitter)) + 1)
            n = int(g.integers(lo, hi))
            ids = g.integers(0, self.vocab, size=n + 1, dtype=np.int64).astype(np.int32)
            i += 1
            yield Sequence(ids[:-1], ids[1:].copy()), {"index": i}

    def _cursor_before(self, after, before):
        return {"index": int(after["index"]) - 1}

    def describe(self) -> dict:
        return {**super().describe(), "vocab": self.vocab, "mean_len": self.mean_len, "seed": self.seed, "eot_id": None}
