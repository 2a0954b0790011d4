"""Token-shard corpora: files with a 1024-byte header (256 int32: magic 20240520, version 1, token count) followed
by uint16 ids (the llm.c shard format).  Default: one sequence per DOCUMENT (split at the delimiter id, which
never appears as an input; the last position of a document targets the delimiter).  ``window=N``: fixed N-token
windows over the whole stream with the global next-token shift.  Epochs wrap indefinitely.
Parity: reference ``src/dataflow_training/data/sources/shards.py``.
"""
from __future__ import annotations

import glob
import os

import numpy as np

from ..sequence import Sequence
from . import DataSource

MAGIC = 20240520
HEADER_BYTES = 1024


def write_shard(path: str, ids) -> None:
    ids = np.asarray(ids)
    if ids.max(initial=0) >= 65536:
        raise ValueError("shard ids must fit uint16")
    head = np.zeros(256, dtype=np.int32)
    head[0], head[1], head[2] = MAGIC, 1, len(ids)
    with open(path, "wb") as f:
        f.write(head.tobytes())
        f.write(ids.astype(np.uint16).tobytes())


def read_shard(path: str) -> np.ndarray:
    head = np.fromfile(path, dtype=np.int32, count=256)
    if len(head) < 256 or head[0] != MAGIC:
        raise ValueError(f"{path}: not a token shard (magic {head[0] if len(head) else None})")
    n = int(head[2])
    ids = np.memmap(path, dtype=np.uint16, mode="r", offset=HEADER_BYTES, shape=(n,))
    return ids


class ShardSource(DataSource):
    scheme = "shards"

    def __init__(self, root: str, window: int | None = None, split: str = "train", delimiter: int = 50256, **kw):
        super().__init__(**kw)
        self.root, self.window, self.split, self.delimiter = root, window, split, int(delimiter)
        pats = [os.path.join(root, f"*{split}*.bin"), os.path.join(root, "*.bin")] if os.path.isdir(root) else [root]
        files: list[str] = []
        for p in pats:
            files = sorted(glob.glob(p))
            if files:
                break
        if not files:
            raise FileNotFoundError(f"no token shards under {root!r} (split {split!r})")
        self.files = files

    def start_cursor(self) -> dict:
        return {"epoch": 0, "shard": 0, "pos": 0}

    def raw(self, cursor):
        epoch, si, pos = int(cursor.get("epoch", 0)), int(cursor.get("shard", 0)), int(cursor.get("pos", 0))
        produced, fresh_pass = 0, (si, pos) == (0, 0)
        while True:
            ids = read_shard(self.files[si])
            n = len(ids)
            if self.window:
                w = self.window
                while pos + w + 1 <= n:
                    chunk = np.asarray(ids[pos:pos + w + 1], dtype=np.int32)
                    pos += w
                    produced += 1
                    yield Sequence(chunk[:-1], chunk[1:].copy()), {"epoch": epoch, "shard": si, "pos": pos}
            else:
                delim = np.flatnonzero(np.asarray(ids[pos:]) == self.delimiter) + pos
                for d in delim:
                    if d > pos:
                        doc = np.asarray(ids[pos:d], dtype=np.int32)
                        nxt = int(d) + 1
                        produced += 1
                        yield Sequence.from_document(doc, self.delimiter), {"epoch": epoch, "shard": si, "pos": nxt}
                    pos = int(d) + 1
            si, pos = si + 1, 0
            if si >= len(self.files):
                if produced == 0 and fresh_pass:       # epochs wrap: shards with nothing usable would be read for ever
                    what = f"no window of {self.window} + 1 tokens fits any shard" if self.window else f"no document ends with the delimiter id {self.delimiter}"
                    raise ValueError(f"no usable sequence in {len(self.files)} shard(s) under {self.root!r}: {what}")
                si, epoch, produced, fresh_pass = 0, epoch + 1, 0, True

    def _cursor_before(self, after, before):
        return dict(before)

    def describe(self) -> dict:
        return {**super().describe(), "root": self.root, "files": len(self.files), "window": self.window,
                "split": self.split, "eot_id": self.delimiter, "vocab": 65536}
