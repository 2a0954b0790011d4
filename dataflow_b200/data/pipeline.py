"""``DataPipeline``: source -> feed -> packer as one object the drivers call.  The factory contract the
drivers use is ``pipeline(cursor | None) -> stepper`` with ``stepper.next_step() -> PackedStep``; a
``DataPipeline`` is its own factory.  ``fast_forward`` resumes checkpoints that carry no cursor by re-packing
on the CPU; ``PrepackedPipeline`` replays steps that were built elsewhere.
Contract parity: reference ``src/dataflow_training/data/pipeline.py:16-131``.
"""
from __future__ import annotations

from typing import Any, Callable, Mapping

from .feed import DataFeed
from .packer import Packer
from .sequence import PackedStep
from .sources import DataSource, resolve_data


class _Stepper:
    def __init__(self, feed: DataFeed, packer: Packer):
        self.feed, self.packer = feed, packer

    def next_step(self) -> PackedStep | None:
        return self.packer.next_step()

    @property
    def stats(self) -> dict:
        st = dict(self.packer.stats)
        st["mean_fill"] = st["content_tokens"] / st["capacity_tokens"] if st["capacity_tokens"] else 0.0
        return st

    def close(self) -> None:
        self.feed.close()


class DataPipeline:
    def __init__(self, source: DataSource | str, tokens_per_round: int, ga_rounds: int, *, max_seqlen: int | None = None,
                 vocab_size: int | None = None, policy: str = "ffd", allow_round_split: bool = False,
                 lookahead: float = 4.0, prefetch_sequences: int = 256, capture: str | None = None):
        self.source = resolve_data(source, vocab_size, max_seqlen) if isinstance(source, str) else source
        self.spec = source if isinstance(source, str) else source.describe().get("scheme", "?")
        self.T, self.R, self.max_seqlen = int(tokens_per_round), int(ga_rounds), max_seqlen
        self.policy, self.split, self.lookahead = policy, allow_round_split, lookahead
        self.prefetch, self.capture = prefetch_sequences, capture
        self.vocab_size = vocab_size

    def __call__(self, cursor: Mapping[str, Any] | None = None) -> _Stepper:
        feed = DataFeed(self.source, self.prefetch, self.capture, (cursor or {}).get("source") if cursor else None)
        packer = Packer(feed, self.T, self.R, self.max_seqlen, self.policy, self.split, self.lookahead,
                        cursor=dict(cursor) if cursor else None)
        return _Stepper(feed, packer)

    def describe(self) -> dict:
        return {"source": self.source.describe(), "tokens_per_round": self.T, "ga_rounds": self.R,
                "max_seqlen": self.max_seqlen, "packing_policy": self.policy, "allow_round_split": self.split,
                "lookahead": self.lookahead}


class PrepackedPipeline:
    """Replays a list of ``PackedStep``s (built by another process, or by a test)."""

    def __init__(self, steps: list[PackedStep]):
        self.steps = list(steps)

    def __call__(self, cursor: Mapping[str, Any] | None = None):
        start = int((cursor or {}).get("step", 0))
        it = iter(self.steps[start:])

        class _S:
            stats: dict = {}

            def next_step(self_inner):
                return next(it, None)

            def close(self_inner):
                pass
        return _S()

    def describe(self) -> dict:
        return {"source": {"scheme": "prepacked"}, "steps": len(self.steps)}


def fast_forward(factory: Callable, steps: int):
    """A stepper positioned after ``steps`` optimizer steps (for checkpoints without a data cursor)."""
    st = factory(None)
    for _ in range(steps):
        if st.next_step() is None:
            break
    return st


def pipeline_from_args(cfg, spec: str | None = None, *, policy: str = "ffd", allow_round_split: bool = False,
                       capture: str | None = None, prefetch_sequences: int = 256) -> DataPipeline:
    """The pipeline of a run config: geometry from ``cfg`` (tokens per round = batch x seq_len), source from the
    ``--data`` spec (default: seeded synthetic documents)."""
    T = int(getattr(cfg, "batch", 1)) * int(cfg.seq_len)
    spec = spec or f"synthetic:mean_len={max(int(cfg.seq_len) // 2, 8)},seed=0"
    return DataPipeline(spec, T, int(cfg.grad_accum_rounds), max_seqlen=int(cfg.seq_len), vocab_size=int(cfg.vocab_size),
                        policy=policy, allow_round_split=allow_round_split, capture=capture,
                        prefetch_sequences=prefetch_sequences)


def legacy_block_pipeline(cfg, root: str, capture: str | None = None) -> DataPipeline:
    """Fixed seq_len windows over a shard corpus in feed order: every round exactly full."""
    T = int(getattr(cfg, "batch", 1)) * int(cfg.seq_len)
    return DataPipeline(f"shards:{root},window={int(cfg.seq_len)}", T, int(cfg.grad_accum_rounds),
                        max_seqlen=int(cfg.seq_len), vocab_size=int(cfg.vocab_size), policy="greedy", capture=capture)
