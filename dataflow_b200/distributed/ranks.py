"""Fleet mode (one dataflowd per rank, driven by a conductor through ``EngineClient``s): per-rank state, one
thread per rank for a lock-step step, and the payload upload of a rank's rounds.
Role parity: reference ``src/dataflow_training/distributed/ranks.py:12-140``.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass
class RankState:
    rank: int
    client: Any                              # EngineClient
    prog_id: str | None = None
    rounds: int = 1
    tokens_per_round: int = 0
    loss_ids: list[str] = field(default_factory=list)
    meta: dict[str, Any] = field(default_factory=dict)


class StepRun(threading.Thread):
    """One rank's ``client.run`` for one optimizer step; join() then read ``.loss`` or ``.error``."""

    def __init__(self, state: RankState, step: int, valid_rows: int, seq_lens: Mapping[int, list[int]] | None = None,
                 extra_args: Mapping[str, Any] | None = None):
        super().__init__(name=f"dataflow-step-rank{state.rank}", daemon=True)
        self.state, self.step = state, step
        self.args = {"step": int(step), "valid_rows": int(valid_rows), **dict(extra_args or {})}
        if seq_lens:
            self.args["seq_lens"] = {str(k): list(v) for k, v in seq_lens.items()}
        self.loss: float | None = None
        self.result: dict | None = None
        self.error: BaseException | None = None

    def run(self) -> None:
        import struct
        try:
            out = self.state.client.run(self.state.prog_id, args=self.args, fetch=self.state.loss_ids)
            self.result = out
            total = 0.0
            for k in self.state.loss_ids:
                raw = out["fetched"][k]               # the daemon decodes 4-byte objects; raw bytes come from older daemons
                total += float(raw) if isinstance(raw, (int, float)) else struct.unpack("<f", raw[:4])[0]
            self.loss = total
        except BaseException as e:       # noqa: BLE001
            self.error = e


def put_rank_rounds(state: RankState, packed, world_rank: int) -> int:
    """Upload this rank's rounds of a packed step (``tokens_0_r`` / ``targets_0_r`` int32 payloads)."""
    n = 0
    for r in range(state.rounds):
        rd = packed.rounds[world_rank * state.rounds + r]
        state.client.put_object(f"tokens_0_{r}", rd.tokens.tobytes())
        state.client.put_object(f"targets_0_{r}", rd.targets.tobytes())
        n += 2 * rd.tokens.nbytes
    return n


def run_step(states: list[RankState], step: int, packed, valid_rows: int | None = None) -> list[float]:
    """Lock step over all ranks: upload, start every rank's run, join, raise the first error."""
    valid = packed.valid_rows if valid_rows is None else valid_rows
    jobs = []
    for s in states:
        put_rank_rounds(s, packed, s.rank)
        sl = {r: packed.seq_lens(True)[s.rank * s.rounds + r] for r in range(s.rounds)}
        jobs.append(StepRun(s, step, valid, sl))
    for j in jobs:
        j.start()
    for j in jobs:
        j.join()
    for j in jobs:
        if j.error is not None:
            raise j.error
    return [j.loss for j in jobs]
