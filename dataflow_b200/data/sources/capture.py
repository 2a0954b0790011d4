"""Capture files: a log of every sequence a feed handed out (after tokenization and the length policy), and the
source that replays one exactly.  Two legs of a comparison (engine vs reference twin, two machines) that read
the same capture provably consume identical data.  Format: a JSON header line, then per sequence one JSON line
``{"n": tokens, "extras": [...]}`` followed by the raw int32 tokens and targets.
Parity: reference ``src/dataflow_training/data/sources/capture.py``.
"""
from __future__ import annotations

import json

import numpy as np

from ..sequence import Sequence
from . import DataSource

CAPTURE_SCHEMA = "dataflow-capture/v1"


class CaptureWriter:
    def __init__(self, path: str, describe: dict | None = None):
        self.f = open(path, "wb")
        self.f.write((json.dumps({"schema": CAPTURE_SCHEMA, "source": describe or {}}) + "\n").encode())
        self.count = 0

    def write(self, seq: Sequence) -> None:
        head = {"n": len(seq), "extras": sorted(seq.extras)}
        self.f.write((json.dumps(head) + "\n").encode())
        self.f.write(seq.tokens.tobytes())
        self.f.write(seq.targets.tobytes())
        for k in sorted(seq.extras):
            a = np.ascontiguousarray(seq.extras[k], dtype=np.float32)
            self.f.write(a.tobytes())
        self.count += 1

    def close(self) -> None:
        self.f.flush()
        self.f.close()


class CaptureSource(DataSource):
    scheme = "capture"
    finite = True

    def __init__(self, path: str):
        super().__init__(None, "whole")
        self.path = path
        with open(path, "rb") as f:
            head = json.loads(f.readline())
        if head.get("schema") != CAPTURE_SCHEMA:
            raise ValueError(f"{path}: not a capture file (schema {head.get('schema')!r})")
        self.recorded = head.get("source", {})

    def start_cursor(self) -> dict:
        return {"index": 0, "offset": 0}

    def raw(self, cursor):
        i, off = int(cursor.get("index", 0)), int(cursor.get("offset", 0))
        with open(self.path, "rb") as f:
            if off:
                f.seek(off)
            else:
                f.readline()
            while True:
                line = f.readline()
                if not line:
                    return
                head = json.loads(line)
                n = int(head["n"])
                tok = np.frombuffer(f.read(4 * n), dtype=np.int32).copy()
                tgt = np.frombuffer(f.read(4 * n), dtype=np.int32).copy()
                extras = {k: np.frombuffer(f.read(4 * n), dtype=np.float32).copy() for k in head.get("extras", [])}
                i += 1
                yield Sequence(tok, tgt, extras), {"index": i, "offset": f.tell()}

    def describe(self) -> dict:
        return {"scheme": "capture", "path": self.path, "recorded": self.recorded,
                "eot_id": self.recorded.get("eot_id"), "vocab": self.recorded.get("vocab")}
