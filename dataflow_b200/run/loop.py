"""The training loop every rank runs: pack the next step's data while the current one executes, write the
rank's rounds into the store, run the step, log, checkpoint.

Data parallel ranks all run the same deterministic pipeline over ``rounds x world`` rounds per step and keep
their own ``rounds`` of it, so no data crosses between ranks and every rank holds the same resume cursor.  The
loss denominator is the job-wide count of real targets.  Role parity: reference
``src/dataflow_training/run/loop.py:115-436`` (there one conductor thread per rank drives a daemon; here one
process per GPU runs this loop and ``torch.distributed`` carries the few scalars that must agree).
"""
from __future__ import annotations

import threading
import time
from typing import Any, Callable, Mapping

import numpy as np

from .driver import RunResult, Trainer


class PackAhead:
    """Builds step ``k + 1`` on a worker thread while step ``k`` runs."""

    def __init__(self, stepper):
        self.stepper = stepper
        self._next = None
        self._thread: threading.Thread | None = None
        self._err: BaseException | None = None
        self._kick()

    def _kick(self) -> None:
        def work():
            try:
                self._next = self.stepper.next_step()
            except BaseException as e:       # noqa: BLE001
                self._err = e
        self._thread = threading.Thread(target=work, name="dataflow-packahead", daemon=True)
        self._thread.start()

    def take(self):
        self._thread.join()
        if self._err is not None:
            raise self._err
        step = self._next
        if step is not None:
            self._kick()
        return step


def _dist():
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            return dist
    except Exception:       # noqa: BLE001
        pass
    return None


def put_rank_rounds(trainer: Trainer, packed, rank: int, rounds: int, row_shard: tuple[int, int] | None = None,
                    first_round: int | None = None) -> tuple[int, dict[int, list[int]], int]:
    """Copy this rank's rounds of a packed step into the store.  Returns (bytes written, seq_lens, local valid rows).
    ``rank``: the DATA rank (which block of ``rounds`` rounds of the step is this rank's).  ``row_shard = (index, count)``:
    sequence parallelism — the ranks of one tensor-parallel group share a data rank, take the SAME rounds and keep their
    slice of rows (the sequence bounds stay those of the whole round: attention sees all rows)."""
    import torch
    nbytes, seq_lens, valid = 0, {}, 0
    for r in range(rounds):
        rd = packed.rounds[(rank * rounds if first_round is None else first_round) + r]
        tk, tg = torch.from_numpy(rd.tokens), torch.from_numpy(rd.targets)
        if row_shard:
            n = len(rd.tokens) // row_shard[1]
            tk, tg = tk[row_shard[0] * n:(row_shard[0] + 1) * n].contiguous(), tg[row_shard[0] * n:(row_shard[0] + 1) * n].contiguous()
        nbytes += trainer.put_round(r, tk, tg)
        b = list(rd.bounds)
        if rd.content < len(rd.tokens):
            b.append(len(rd.tokens))          # the tail rides as one masked segment: defined values, zero loss
        seq_lens[r] = b
        valid += rd.valid_rows
    return nbytes, seq_lens, valid


def train_loop(trainer: Trainer, factory: Callable, steps: int, *, cursor: Mapping[str, Any] | None = None,
               start_step: int = 0, losses: list[float] | None = None, checkpoint_every: int = 0,
               checkpoint_dir: str | None = None, keep_last: int | None = None, seed: int = 0,
               launch: Mapping[str, Any] | None = None, log: Callable[[str], None] | None = print,
               on_step: Callable[[int, float, Any], None] | None = None, rank_rounds: list[int] | None = None,
               window=None, checkpoint_redundancy: int | None = None) -> RunResult:
    """Run optimizer steps ``start_step + 1 .. steps``.  ``factory(cursor)`` builds the data stepper; its packed
    steps must hold ``trainer.rounds x world`` rounds of ``trainer.T`` tokens."""
    from .checkpointing import save_checkpoint
    dist = _dist()
    rank = dist.get_rank() if dist else 0
    world = dist.get_world_size() if dist else 1
    # data-parallel ranks (fsdp / zero / ep) consume different rounds; tensor-parallel ranks share them and split the rows
    tp = int((trainer.program.metadata or {}).get("tp", 1))
    row_shard = (rank % tp, tp) if tp > 1 else None
    data_world = world // tp if row_shard else world          # > 1 with tp: a dp x tp mesh, replicas consume different rounds
    data_rank = rank // tp if row_shard else rank
    # weighted data parallelism: rank r runs rank_rounds[r] rounds of every step
    job_rounds = sum(rank_rounds) if rank_rounds else trainer.rounds * data_world
    first_round = sum(rank_rounds[:rank]) if rank_rounds else None
    stepper = factory(dict(cursor) if cursor else None)
    ahead = PackAhead(stepper)
    res = RunResult(losses=list(losses or []), tokens_per_step=trainer.T * (job_rounds if rank_rounds else trainer.rounds * world),     # T is this rank's rows of a round
                    meta={"family": trainer.fam.name, "preset": getattr(trainer.cfg, "name", ""), "world": world,
                          "plan_makespan_us": trainer.planned.makespan_us, "policy": trainer.planned.policy,
                          "peak_fast_bytes": trainer.planned.peak_fast_bytes,
                          "data": getattr(factory, "describe", lambda: {})()})
    trainer.step_index = start_step
    content_total = 0
    try:
        for s in range(start_step, steps):
            packed = ahead.take()
            if packed is None:
                if log and rank == 0:
                    log(f"data source exhausted after {s} steps")
                break
            if len(packed.rounds) != job_rounds:
                raise ValueError(f"packed step has {len(packed.rounds)} rounds, the job consumes {job_rounds}")
            if window:
                window.before(s + 1, trainer)
            t0 = time.perf_counter()
            _, seq_lens, valid = put_rank_rounds(trainer, packed, data_rank, trainer.rounds, row_shard, first_round)
            total_valid = packed.valid_rows          # every rank packed the whole job's step: no exchange needed
            loss = trainer.step(None, seq_lens=seq_lens, valid_rows=max(total_valid, 1))
            if dist:
                import torch
                t = torch.tensor([loss], dtype=torch.float64, device="cuda" if trainer.device is not None else "cpu")
                dist.all_reduce(t)
                loss = float(t[0])
            dt = time.perf_counter() - t0
            if window:
                window.after(s + 1, trainer)
            res.losses.append(loss)
            res.step_wall_s.append(dt)
            content_total += packed.content_tokens
            if log and rank == 0:
                log(f"step {s + 1:5d}  loss {loss:.4f}  {packed.content_tokens / dt:,.0f} tok/s  fill {packed.fill:.3f}  "
                    f"lr {_lr(trainer, s + 1):.3e}")
            if on_step is not None:
                on_step(s + 1, loss, packed)
            if checkpoint_every and checkpoint_dir and (s + 1) % checkpoint_every == 0:
                save_checkpoint(trainer, checkpoint_dir, s + 1, seed=seed, keep_last=keep_last, launch=launch,
                                redundancy=checkpoint_redundancy,
                                client_payload={"losses": res.losses, "cursor": dict(packed.cursor_after)},
                                summary={"last_loss": loss, "steps_recorded": len(res.losses)})
    finally:
        if hasattr(stepper, "close"):
            stepper.close()
    st = getattr(stepper, "stats", None)
    if st:
        res.meta["data_stats"] = dict(st)
    res.meta["content_tokens"] = content_total
    return res


def _lr(trainer: Trainer, step: int) -> float:
    from ..blocks.optim import lr_at
    return lr_at(trainer.hyper, step)


def reference_loop(family: str, cfg, factory: Callable, steps: int, hyper: Mapping[str, Any], *, seed: int = 0,
                   views_of=None, log: Callable[[str], None] | None = print) -> RunResult:
    """The pure-torch twin on the same packed data (fp32 autograd + torch.optim.AdamW): the oracle curve."""
    import torch
    from ..blocks.optim import lr_at
    from ..models.families import resolve_family
    fam = resolve_family(family)
    twin = fam.twin(cfg)
    if views_of is not None:
        twin.load_state_dict(fam.bridge(cfg, views_of))
    decay = [p for _, p in twin.named_parameters() if p.dim() >= 2]
    plain = [p for _, p in twin.named_parameters() if p.dim() < 2]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": hyper.get("weight_decay", 0.0)},
                             {"params": plain, "weight_decay": 0.0}], lr=hyper.get("lr", 3e-4),
                            betas=(hyper.get("beta1", 0.9), hyper.get("beta2", 0.95)), eps=hyper.get("eps", 1e-8))
    stepper = factory(None)
    res = RunResult(meta={"family": family, "leg": "reference"})
    try:
        for s in range(steps):
            packed = stepper.next_step()
            if packed is None:
                break
            for g in opt.param_groups:
                g["lr"] = lr_at(hyper, s + 1)
            opt.zero_grad()
            total = 0.0
            t0 = time.perf_counter()
            denom = max(packed.valid_rows, 1)
            for rd in packed.rounds:
                tk = torch.from_numpy(rd.tokens[:rd.content].astype(np.int64))
                tg = torch.from_numpy(rd.targets[:rd.content].astype(np.int64))
                l = twin.loss(tk, tg, list(rd.bounds), total_rows=denom)
                l.backward()
                total += float(l.detach())
            opt.step()
            res.losses.append(total)
            res.step_wall_s.append(time.perf_counter() - t0)
            res.tokens_per_step = sum(len(r.tokens) for r in packed.rounds)
            if log:
                log(f"ref step {s + 1:5d}  loss {total:.4f}")
    finally:
        if hasattr(stepper, "close"):
            stepper.close()
    return res
