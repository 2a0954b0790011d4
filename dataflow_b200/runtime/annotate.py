"""Annotators: who is told when the executor opens and closes a range (one per task launch, one per transfer issue).

``NvtxAnnotator``      NVTX ranges for a profiler's timeline; off (pure no-ops) until ``start_capture()``.
``RecordingAnnotator`` keeps the ranges in a list: tests, and tools that want the launch order without a profiler.
``annotate_rename``    (an argument of ``Engine.execute``) maps an id to the name that is SHOWN — ``(name, kind) -> str``
                       with kind ``"task"`` or ``"transfer"`` — so a timeline can carry readable labels (``L12 fwd r3``)
                       while programs keep their ids.  It never changes what runs.
Role parity: reference ``src/dataflow/runtime/device/annotate.py`` and the ``annotate_rename`` argument of its engine
(``src/dataflow/runtime/engine.py:522,858``; ``runtime/transfers.py:199``).
"""
from __future__ import annotations

import os
from typing import Callable


class NoopAnnotator:
    enabled = False

    def range_push(self, name: str) -> None:
        pass

    def range_pop(self) -> None:
        pass


class RecordingAnnotator:
    """Every push and pop, in order: ``events`` holds ``("push", name)`` / ``("pop", name)``; ``depth_ok()`` says whether
    every range that was opened has been closed."""
    enabled = True

    def __init__(self):
        self.events: list[tuple[str, str]] = []
        self._open: list[str] = []

    def range_push(self, name: str) -> None:
        self._open.append(name)
        self.events.append(("push", name))

    def range_pop(self) -> None:
        self.events.append(("pop", self._open.pop() if self._open else "?"))

    def depth_ok(self) -> bool:
        return not self._open

    def names(self, prefix: str = "") -> list[str]:
        return [n for k, n in self.events if k == "push" and n.startswith(prefix)]


class NvtxAnnotator:
    """NVTX ranges through the native module; ``enabled`` follows the capture window."""

    def __init__(self, enabled: bool = False):
        from . import _runtime
        self._rt = _runtime
        self.enabled = bool(enabled)

    def start_capture(self) -> None:
        self.enabled = True

    def stop_capture(self) -> None:
        self.enabled = False

    def range_push(self, name: str) -> None:
        if self.enabled:
            self._rt.nvtx_push(name)

    def range_pop(self) -> None:
        if self.enabled:
            self._rt.nvtx_pop()


def annotator_from_env():
    """``DATAFLOW_ANNOTATE``: ``nvtx`` (ranges from the first task on), ``record``, anything else / unset = none."""
    kind = os.environ.get("DATAFLOW_ANNOTATE", "")
    if kind == "nvtx":
        return NvtxAnnotator(enabled=True)
    if kind == "record":
        return RecordingAnnotator()
    return None


def make_hook(annotator, rename: Callable[[str, str], str] | None):
    """The ``(name, push)`` callable the native executor calls; transfers arrive as ``xfer:<name>``."""
    if annotator is None:
        return None

    def hook(name: str, push: bool) -> None:
        if not getattr(annotator, "enabled", True):
            return
        if not push:
            annotator.range_pop()
            return
        kind = "task"
        if name.startswith("xfer:"):
            kind, name = "transfer", name[5:]
        annotator.range_push(rename(name, kind) if rename is not None else name)
    return hook
