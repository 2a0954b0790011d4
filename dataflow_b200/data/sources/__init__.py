"""Data sources.  One contract: ``sequences(cursor)`` is a pure function of (constructor arguments, cursor)
— two iterations from equal cursors yield byte-identical sequences — and yields ``(Sequence, cursor_after)``
pairs; ``describe()`` reports JSON-clean facts for run metadata.  The over-long policy (``exclude`` | ``trim`` |
``chunk`` | ``whole``) is applied at the source.  ``resolve_data("scheme:main,k=v,...")`` builds one from a CLI
spec.  Contract parity: reference ``src/dataflow_training/data/sources/__init__.py``.
"""
from __future__ import annotations

from typing import Any, Iterator, Mapping

from ..sequence import Sequence

LONG_POLICIES = ("exclude", "trim", "chunk", "whole")


class DataSource:
    scheme = "?"
    finite = False

    def __init__(self, max_seqlen: int | None = None, long_policy: str = "exclude"):
        if long_policy not in LONG_POLICIES:
            raise ValueError(f"long_policy must be one of {LONG_POLICIES}, got {long_policy!r}")
        self.max_seqlen = max_seqlen
        self.long_policy = long_policy

    # -- subclass surface
    def start_cursor(self) -> dict:
        return {}

    def raw(self, cursor: Mapping[str, Any]) -> Iterator[tuple[Sequence, dict]]:
        raise NotImplementedError

    def describe(self) -> dict:
        return {"scheme": self.scheme, "max_seqlen": self.max_seqlen, "long_policy": self.long_policy}

    # -- policy
    def sequences(self, cursor: Mapping[str, Any] | None = None) -> Iterator[tuple[Sequence, dict]]:
        cur = dict(cursor) if cursor else self.start_cursor()
        part0 = int(cur.pop("_part", 0))
        first = True
        for seq, after in self.raw(cur):
            skip = part0 if first else 0
            first = False
            m = self.max_seqlen
            if not m or len(seq) <= m or self.long_policy == "whole":
                yield seq, after
            elif self.long_policy == "exclude":
                continue
            elif self.long_policy == "trim":
                yield seq.slice(0, m), after
            else:   # chunk: pieces of max_seqlen; the cursor of a middle piece re-enters the same document
                n = (len(seq) + m - 1) // m
                for k in range(skip, n):
                    c = after if k == n - 1 else {**self._cursor_before(after, cur), "_part": k + 1}
                    yield seq.slice(k * m, min((k + 1) * m, len(seq))), c
            cur = after

    def _cursor_before(self, after: Mapping[str, Any], before: Mapping[str, Any]) -> dict:
        return dict(before)


def parse_spec(spec: str) -> tuple[str, str, dict[str, str]]:
    scheme, _, rest = spec.partition(":")
    parts = rest.split(",") if rest else [""]
    main = parts[0] if parts and "=" not in parts[0] else ""
    kv = {}
    for p in parts[(1 if main or (parts and "=" not in parts[0]) else 0):]:
        if not p:
            continue
        k, _, v = p.partition("=")
        kv[k.strip()] = v.strip()
    return scheme, main, kv


def resolve_data(spec: str, vocab_size: int | None = None, max_seqlen: int | None = None) -> DataSource:
    scheme, main, kv = parse_spec(spec)
    lp = kv.pop("long_policy", "exclude")
    ms = int(kv.pop("max_seqlen", max_seqlen or 0)) or None
    if scheme == "synthetic":
        from .synthetic import SyntheticSource
        return SyntheticSource(vocab=int(kv.pop("vocab", vocab_size or 50257)), mean_len=int(kv.pop("mean_len", 512)),
                               seed=int(kv.pop("seed", 0)), max_seqlen=ms, long_policy=lp, **_rest(kv))
    if scheme == "shards":
        from .shards import ShardSource
        return ShardSource(main or kv.pop("root", ""), window=int(kv.pop("window", 0)) or None, split=kv.pop("split", "train"),
                           max_seqlen=ms, long_policy=lp, **_rest(kv))
    if scheme in ("jsonl", "txt"):
        from .jsonl import TextSource
        return TextSource(main, tokenizer=kv.pop("tokenizer", "bytes"), fmt=scheme, field=kv.pop("field", "text"),
                          delimiter=kv.pop("delimiter", "\n\n").encode().decode("unicode_escape"),
                          vocab_size=vocab_size, max_seqlen=ms, long_policy=lp, **_rest(kv))
    if scheme == "parquet":
        from .parquet import ParquetSource
        return ParquetSource(main, tokenizer=kv.pop("tokenizer", "bytes"), column=kv.pop("column", "text"),
                             vocab_size=vocab_size, max_seqlen=ms, long_policy=lp, **_rest(kv))
    if scheme == "capture":
        from .capture import CaptureSource
        return CaptureSource(main, **_rest(kv))
    raise KeyError(f"unknown data scheme {scheme!r} (synthetic | shards | jsonl | txt | parquet | capture)")


def _rest(kv: dict) -> dict:
    if kv:
        raise KeyError(f"unknown data spec keys {sorted(kv)}")
    return {}
