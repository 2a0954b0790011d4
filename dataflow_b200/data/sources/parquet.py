"""Parquet text column, streamed one row group at a time and tokenized at ingest.
Parity: reference ``src/dataflow_training/data/sources/parquet.py``.
"""
from __future__ import annotations

import glob

import numpy as np

from ..sequence import Sequence
from ..tokenizers import resolve_tokenizer
from . import DataSource


class ParquetSource(DataSource):
    scheme = "parquet"

    def __init__(self, pattern: str, tokenizer: str = "bytes", column: str = "text", vocab_size: int | None = None, **kw):
        super().__init__(**kw)
        self.files = sorted(glob.glob(pattern))
        if not self.files:
            raise FileNotFoundError(f"no files match {pattern!r}")
        self.tok = resolve_tokenizer(tokenizer)
        self.column = column
        if vocab_size is not None and self.tok.vocab_size > vocab_size:
            raise ValueError(f"tokenizer {tokenizer!r} has {self.tok.vocab_size} ids, the model's vocabulary is {vocab_size}")

    def start_cursor(self) -> dict:
        return {"epoch": 0, "file": 0, "group": 0, "row": 0}

    def raw(self, cursor):
        import pyarrow.parquet as pq
        epoch, fi = int(cursor.get("epoch", 0)), int(cursor.get("file", 0))
        gi, ri = int(cursor.get("group", 0)), int(cursor.get("row", 0))
        produced, fresh_pass = 0, (fi, gi, ri) == (0, 0, 0)
        while True:
            pf = pq.ParquetFile(self.files[fi])
            for g in range(gi, pf.num_row_groups):
                col = pf.read_row_group(g, columns=[self.column]).column(self.column).to_pylist()
                for k in range(ri if g == gi else 0, len(col)):
                    text = col[k]
                    if not text:
                        continue
                    ids = np.asarray(self.tok.encode(text), dtype=np.int32)
                    if len(ids) >= 2:
                        produced += 1
                        yield Sequence.from_document(ids, self.tok.eot_id), {"epoch": epoch, "file": fi, "group": g, "row": k + 1}
            fi, gi, ri = fi + 1, 0, 0
            if fi >= len(self.files):
                if produced == 0 and fresh_pass:       # epochs wrap: a corpus with nothing usable would be read for ever
                    raise ValueError(f"no usable document in {len(self.files)} parquet file(s): column {self.column!r} holds no text of at least two tokens")
                fi, epoch, produced, fresh_pass = 0, epoch + 1, 0, True

    def describe(self) -> dict:
        return {**super().describe(), "files": len(self.files), "column": self.column, "tokenizer": self.tok.describe(),
                "eot_id": self.tok.eot_id, "vocab": self.tok.vocab_size}
