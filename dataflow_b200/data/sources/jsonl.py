"""Text sources tokenized at ingest: ``jsonl`` (one document per JSON line, ``field`` names the text; records
with ``instruction`` / ``output`` keep the prompt masked out of the loss) and ``txt`` (delimiter-split plain
text).  Files of the glob are read in sorted order; epochs wrap.  Token ids are checked against the run's
vocabulary.  Parity: reference ``src/dataflow_training/data/sources/jsonl.py``.
"""
from __future__ import annotations

import glob
import json

import numpy as np

from ..sequence import IGNORE_INDEX, Sequence
from ..tokenizers import resolve_tokenizer
from . import DataSource


class TextSource(DataSource):
    scheme = "jsonl"

    def __init__(self, pattern: str, tokenizer: str = "bytes", fmt: str = "jsonl", field: str = "text",
                 delimiter: str = "\n\n", vocab_size: int | None = None, **kw):
        super().__init__(**kw)
        self.scheme = fmt
        self.files = sorted(glob.glob(pattern))
        if not self.files:
            raise FileNotFoundError(f"no files match {pattern!r}")
        self.tok = resolve_tokenizer(tokenizer)
        self.field, self.delimiter, self.vocab_size = field, delimiter, vocab_size
        if vocab_size is not None and self.tok.vocab_size > vocab_size:
            raise ValueError(f"tokenizer {tokenizer!r} has {self.tok.vocab_size} ids, the model's vocabulary is {vocab_size}")

    def start_cursor(self) -> dict:
        return {"epoch": 0, "file": 0, "record": 0}

    def _records(self, path: str):
        if self.scheme == "jsonl":
            with open(path, "r", encoding="utf-8") as f:
                for lineno, line in enumerate(f, 1):
                    line = line.strip()
                    if not line:
                        continue
                    try:
                        rec = json.loads(line)
                    except ValueError as e:
                        raise ValueError(f"{path}:{lineno}: not a JSON document ({e})") from None
                    if not isinstance(rec, dict):
                        raise ValueError(f"{path}:{lineno}: a record must be a JSON object, this line is a {type(rec).__name__}")
                    yield rec
        else:
            with open(path, "r", encoding="utf-8") as f:
                for part in f.read().split(self.delimiter):
                    if part.strip():
                        yield {"text": part}

    def _encode(self, rec) -> Sequence | None:
        eot = self.tok.eot_id
        if "instruction" in rec and "output" in rec and self.field not in rec:
            p, r = self.tok.encode(rec["instruction"]), self.tok.encode(rec["output"])
            ids = np.asarray(p + r, dtype=np.int32)
            if len(ids) < 2:
                return None
            seq = Sequence.from_document(ids, eot)
            seq.targets[:max(len(p) - 1, 0)] = IGNORE_INDEX       # the prompt is context, not loss
            return seq
        text = rec.get(self.field if self.scheme == "jsonl" else "text")
        if not text:
            return None
        ids = np.asarray(self.tok.encode(text), dtype=np.int32)
        if len(ids) < 2:
            return None
        return Sequence.from_document(ids, eot)

    def raw(self, cursor):
        epoch, fi, ri = int(cursor.get("epoch", 0)), int(cursor.get("file", 0)), int(cursor.get("record", 0))
        produced = 0                    # documents of the current pass over the files
        started = (fi, ri)
        while True:
            for k, rec in enumerate(self._records(self.files[fi])):
                if k < ri:
                    continue
                seq = self._encode(rec)
                if seq is not None:
                    produced += 1
                    yield seq, {"epoch": epoch, "file": fi, "record": k + 1}
            fi, ri = fi + 1, 0
            if fi >= len(self.files):
                if produced == 0 and started == (0, 0):
                    # epochs wrap: without this a corpus with nothing usable in it would be read for ever
                    what = f"field {self.field!r}" if self.scheme == "jsonl" else "text"
                    raise ValueError(f"no usable document in {len(self.files)} file(s) matching the source ({what} of at least two tokens)")
                fi, epoch, produced, started = 0, epoch + 1, 0, (0, 0)

    def describe(self) -> dict:
        return {**super().describe(), "files": len(self.files), "tokenizer": self.tok.describe(), "eot_id": self.tok.eot_id,
                "vocab": self.tok.vocab_size}
