"""``DataFeed``: hands out a source's sequences in source order through one background ingest worker and a
bounded queue (back-pressure blocks the worker), with ``requeue`` for packer remainders, an optional capture
log of everything handed out, and a JSON-able cursor that names the position right after the last sequence the
consumer KEPT.  ``prefetch_sequences=0`` is the synchronous path; both paths hand out identical sequences.
Contract parity: reference ``src/dataflow_training/data/feed.py:52-234``.
"""
from __future__ import annotations

import queue
import threading
from collections import deque
from typing import Any, Mapping

from .sequence import Sequence
from .sources import DataSource
from .sources.capture import CaptureWriter

_END = object()


class IngestWorker(threading.Thread):
    def __init__(self, source: DataSource, cursor, depth: int):
        super().__init__(name="dataflow-ingest", daemon=True)
        self.q: "queue.Queue[Any]" = queue.Queue(maxsize=max(depth, 1))
        self.source, self.cursor = source, cursor
        self._halt = threading.Event()

    def run(self) -> None:
        try:
            for item in self.source.sequences(self.cursor):
                while not self._halt.is_set():
                    try:
                        self.q.put(item, timeout=0.1)
                        break
                    except queue.Full:
                        continue
                if self._halt.is_set():
                    return
            self.q.put(_END)
        except BaseException as e:         # noqa: BLE001  surfaced on the consumer's next call
            self.q.put(e)

    def stop(self) -> None:
        self._halt.set()


class DataFeed:
    def __init__(self, source: DataSource, prefetch_sequences: int = 256, capture: str | None = None,
                 start_cursor: Mapping[str, Any] | None = None):
        self.source = source
        self._cursor = dict(start_cursor) if start_cursor else source.start_cursor()
        self._front: deque[tuple[Sequence, dict | None]] = deque()     # requeued sequences lead the line
        self._capture = CaptureWriter(capture, source.describe()) if capture else None
        self._worker = None
        self._iter = None
        self._exhausted = False
        self.handed_out = 0
        if prefetch_sequences > 0:
            self._worker = IngestWorker(source, dict(self._cursor), prefetch_sequences)
            self._worker.start()
        else:
            self._iter = iter(source.sequences(dict(self._cursor)))

    def _pull(self):
        if self._exhausted:
            return None
        if self._worker is not None:
            item = self._worker.q.get()
            if item is _END:
                self._exhausted = True
                return None
            if isinstance(item, BaseException):
                self._exhausted = True
                raise item
            return item
        try:
            return next(self._iter)
        except StopIteration:
            self._exhausted = True
            return None

    def next_sequence(self) -> tuple[Sequence, dict | None] | None:
        """The next sequence and the cursor right after it (``None`` cursor for a requeued piece that is not
        the tail of its source sequence); ``None`` when a finite source is exhausted."""
        if self._front:
            return self._front.popleft()
        return self._pull()

    def keep(self, seq: Sequence) -> None:
        """The consumer commits to this (piece of a) sequence: it is logged to the capture."""
        if self._capture is not None:
            self._capture.write(seq)
        self.handed_out += 1

    def requeue(self, items: list[tuple[Sequence, dict | None]]) -> None:
        for it in reversed(items):
            self._front.appendleft(it)

    def cursor(self) -> dict:
        """The source cursor this feed was started at (consumers track their own progress from it)."""
        return dict(self._cursor)

    def close(self) -> None:
        if self._worker is not None:
            self._worker.stop()
        if self._capture is not None:
            self._capture.close()
            self._capture = None
