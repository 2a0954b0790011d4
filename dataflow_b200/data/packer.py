"""``Packer``: groups a feed's sequences into the fixed rounds of optimizer steps.

``policy="ffd"`` (default) pulls a lookahead window (``lookahead`` x the step's token budget) and places it
first-fit-decreasing, every round as full as possible; what fits nowhere goes back to the front of the feed in
pull order and leads the next step.  ``policy="greedy"`` fills in feed order and defers at the first non-fit.
``allow_round_split`` lets a sequence split at a round edge so rounds are always exactly full (the fixed-token
legacy packing).  Under-full rounds keep their planner size; ``bounds`` stop at the content edge.

Resume exactness: the cursor stored with a step is only advanced past sequences that every earlier step has
fully consumed, and the step records which pulled sequences it skipped, so ``Packer(..., cursor=step.cursor_after)``
continues with byte-identical steps.  Contract parity: reference ``src/dataflow_training/data/packer.py:71-188``.
"""
from __future__ import annotations

import numpy as np

from .feed import DataFeed
from .sequence import IGNORE_INDEX, PackedRound, PackedStep, Sequence


class Packer:
    def __init__(self, feed: DataFeed, tokens_per_round: int, ga_rounds: int, max_seqlen: int | None = None,
                 policy: str = "ffd", allow_round_split: bool = False, lookahead: float = 4.0, filler_token: int = 0,
                 cursor: dict | None = None):
        """``cursor``: a ``PackedStep.cursor_after`` to continue from (the feed must have been started at
        ``cursor["source"]``; ``packer_from_cursor`` does both)."""
        if policy not in ("ffd", "greedy"):
            raise ValueError(f"packing policy must be ffd or greedy, got {policy!r}")
        self.feed, self.T, self.R = feed, int(tokens_per_round), int(ga_rounds)
        self.max_seqlen = max_seqlen or self.T
        self.policy, self.split, self.lookahead, self.filler = policy, allow_round_split, lookahead, filler_token
        self.stats = {"steps": 0, "content_tokens": 0, "capacity_tokens": 0, "min_fill": 1.0}
        # pulls are numbered from the base: the feed position before the oldest sequence not fully consumed
        self._pending: list[tuple[Sequence, int]] = []       # (what is left of the sequence, pull id)
        self._cursor_after: dict[int, dict | None] = {}      # pull id -> source cursor right after it
        self._done: set[int] = set()                         # consumed pull ids at or beyond the base
        self._partial: dict[int, int] = {}                   # pull id -> tokens already consumed (round split)
        self._next_id = 0
        self._base_id = 0
        self._base_cursor = dict((cursor or {}).get("source") or feed.cursor())
        self._resume_skip = set(int(x) for x in (cursor or {}).get("skip", ()))
        self._resume_partial = {int(k): int(v) for k, v in ((cursor or {}).get("partial") or {}).items()}
        self.step_index = int((cursor or {}).get("step", 0))

    # -- pulling
    def _pull_until(self, want_tokens: int) -> None:
        have = sum(len(s) for s, _ in self._pending)
        while have < want_tokens:
            item = self.feed.next_sequence()
            if item is None:
                break
            seq, cur = item
            pid = self._next_id
            self._next_id += 1
            self._cursor_after[pid] = cur
            if pid in self._resume_skip:           # an earlier step (before the resume point) consumed it
                self._done.add(pid)
                continue
            cut = self._resume_partial.get(pid, 0)
            if cut:
                seq = seq.slice(cut, len(seq))
                self._partial[pid] = cut
            if len(seq) > self.T and not self.split:
                seq = seq.slice(0, self.T)         # fits no round: trimmed (sources normally enforce max_seqlen)
            self._pending.append((seq, pid))
            have += len(seq)

    def next_step(self) -> PackedStep | None:
        T, R = self.T, self.R
        rounds: list[list[Sequence]] = [[] for _ in range(R)]
        room = [T] * R
        used: list[int] = []
        if self.split:
            self._pull_until(T * R)
            r = 0
            k = 0
            while r < R and k < len(self._pending):
                seq, pid = self._pending[k]
                n = len(seq)
                if n <= room[r]:
                    rounds[r].append(seq)
                    room[r] -= n
                    used.append(k)
                    k += 1
                else:
                    take = room[r]
                    if take:
                        rounds[r].append(seq.slice(0, take))
                        self._partial[pid] = self._partial.get(pid, 0) + take
                    self._pending[k] = (seq.slice(take, n), pid)
                    room[r] = 0
                if room[r] == 0:
                    r += 1
        elif self.policy == "greedy":
            self._pull_until(T * R)
            r = 0
            for k, (seq, pid) in enumerate(self._pending):
                while r < R and len(seq) > room[r]:
                    r += 1
                if r >= R:
                    break
                rounds[r].append(seq)
                room[r] -= len(seq)
                used.append(k)
        else:
            self._pull_until(int(T * R * self.lookahead))
            order = sorted(range(len(self._pending)), key=lambda k: (-len(self._pending[k][0]), k))
            placed: dict[int, int] = {}
            for k in order:
                n = len(self._pending[k][0])
                for r in range(R):
                    if n <= room[r]:
                        placed[k] = r
                        room[r] -= n
                        break
            for k in sorted(placed):               # inside a round: feed order
                rounds[placed[k]].append(self._pending[k][0])
                used.append(k)
        if not any(rounds):
            return None
        for rd in rounds:
            for seq in rd:
                self.feed.keep(seq)
        used_set = set(used)
        for k in used:
            pid = self._pending[k][1]
            self._done.add(pid)
            self._partial.pop(pid, None)
        self._pending = [p for k, p in enumerate(self._pending) if k not in used_set]
        self.step_index += 1
        step = PackedStep([self._finish(rd) for rd in rounds], self._cursor(), self.step_index - 1)
        st = self.stats
        st["steps"] += 1
        st["content_tokens"] += step.content_tokens
        st["capacity_tokens"] += T * R
        st["min_fill"] = min(st["min_fill"], step.fill)
        return step

    # -- cursor
    def _cursor(self) -> dict:
        while self._base_id in self._done:
            cur = self._cursor_after.pop(self._base_id)
            if cur is not None:
                self._base_cursor = dict(cur)
            self._done.discard(self._base_id)
            self._base_id += 1
            # ids in a resumed cursor were relative to the old base: keep them relative to the moving one
        out = {"source": dict(self._base_cursor), "step": self.step_index,
               "skip": sorted(i - self._base_id for i in self._done),
               "partial": {str(i - self._base_id): n for i, n in sorted(self._partial.items())}}
        return out

    def _finish(self, seqs: list[Sequence]) -> PackedRound:
        T = self.T
        tok = np.full(T, self.filler, dtype=np.int32)
        tgt = np.full(T, IGNORE_INDEX, dtype=np.int32)
        bounds = [0]
        pos = 0
        for s in seqs:
            n = len(s)
            # a segment longer than max_seqlen (round-split tails of whole documents) restarts positions inside it
            for a in range(0, n, self.max_seqlen):
                b = min(a + self.max_seqlen, n)
                tok[pos + a:pos + b] = s.tokens[a:b]
                tgt[pos + a:pos + b] = s.targets[a:b]
                bounds.append(pos + b)
            pos += n
        return PackedRound(tok, tgt, bounds, pos)
