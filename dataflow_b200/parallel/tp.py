"""Tensor parallelism with sequence parallelism inside one NVSwitch box.

Activations between blocks are sharded by rows (tokens); a column-parallel linear all-gathers them and a
row-parallel linear reduce-scatters its output.  ``TpGroup`` gives both as ONE kernel each
(``ops/csrc/gemm_tp.cu``): ``ag_gemm`` pulls the peers' rows over NVLink from inside the GEMM while the first
panels are already multiplying, ``gemm_rs`` stores each finished tile straight into the owner's memory and the
same kernel reduces the arrived partials.  A ``collective`` lane (``torch.distributed`` all-gather / reduce-
scatter around a library matmul) is the baseline and the oracle of the tests.

Every rank allocates the same *symmetric workspace* and maps the peers' through CUDA IPC: rendezvous words, the
row buffer peers read (``x``), the gathered operand, and the reduce-scatter staging.
The reference's tensor-parallel lane (``--tp-mlp``) all-reduces partial outputs through NCCL
(``src/dataflow_training/model_families/llama3/blocks.py:91-128``); it has no sequence parallelism and no fused kernels.
"""
from __future__ import annotations

import os
from typing import Any
from .group_abi import GroupCollectives

CTRL_BYTES = 1 << 18          # rendezvous words, handed out per operand shape (see ``_words``)


class TpGroup(GroupCollectives):
    def __init__(self, rank: int, world: int, device: int | None, *, max_rows: int, max_k: int, max_n: int,
                 lane: str | None = None, timeout_s: float = 30.0, pg=None):
        """``max_rows``: rows per rank (the sequence shard); ``max_k`` / ``max_n``: widest gathered operand and widest
        reduce-scattered output this group will see (they size the workspace).  ``pg``: the ``torch.distributed`` process
        group of the members when they are a subset of the job (a dp x tp mesh); ``rank`` is the rank inside it."""
        self.rank, self.world, self.device, self.pg = rank, world, device, pg
        self.lane = lane or os.environ.get("DATAFLOW_TP_LANE") or ("p2p" if device is not None else "collective")
        self.timeout_s = timeout_s
        self.max_rows, self.max_k, self.max_n = int(max_rows), int(max_k), int(max_n)
        self.x_bytes = self.max_rows * self.max_k * 2
        self.gathered_bytes = self.world * self.x_bytes
        self.stage_bytes = self.world * self.max_rows * self.max_n * 2
        self.off_gathered = CTRL_BYTES
        self.off_stage = self.off_gathered + _up(self.gathered_bytes)
        self.ws_bytes = self.off_stage + _up(self.stage_bytes)
        self.ws: list[int] = []
        self.backend = None
        self._shapes: dict[tuple, dict] = {}
        self._ctrl_used = 0
        self.name = "tp"

    # -- set-up
    def attach(self, backend) -> None:
        if self.lane != "p2p":
            return
        import torch
        import torch.distributed as dist
        backend = getattr(backend, "backend", backend)          # a Trainer hands itself over
        if self.ws:
            return
        self.backend = backend
        self.base = backend.device_alloc_zeroed(self.ws_bytes)
        handles: list[Any] = [None] * self.world
        dist.all_gather_object(handles, backend.ipc_handle(self.base), group=self.pg)
        self.ws = [self.base if r == self.rank else backend.ipc_open(h) for r, h in enumerate(handles)]
        dev = torch.device("cuda", self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=dev)
        self.done = torch.zeros(1, dtype=torch.int32, device=dev)
        dist.barrier(group=self.pg)

    def close(self) -> None:
        if self.lane == "p2p" and self.backend is not None and self.ws:
            import torch
            torch.cuda.synchronize(self.device)
            for r, p in enumerate(self.ws):
                if r != self.rank:
                    self.backend.ipc_close(p)
            self.backend.device_free(self.base)
            self.ws = []

    def check(self) -> None:
        if self.lane == "p2p":
            code = int(self.err.item())
            if code:
                self.err.zero_()
                raise RuntimeError(f"fused tensor-parallel kernel gave up: phase {code >> 8}, peer/rank {code & 255}")

    def _words(self, key: tuple, nwords: int) -> dict:
        """Rendezvous words of one operand shape.  Counters only grow (target = per-launch increment x launches of
        THIS shape), so every shape gets its own words; all ranks issue the same calls in the same order, hence
        hand out the same offsets."""
        st = self._shapes.get(key)
        if st is None:
            import torch
            nbytes = (nwords * 4 + 255) // 256 * 256
            if self._ctrl_used + nbytes > CTRL_BYTES:
                raise RuntimeError("tensor-parallel group ran out of rendezvous words (too many distinct operand shapes)")
            st = {"off": self._ctrl_used, "seq": 0,
                  "flags": torch.zeros(8, dtype=torch.int32, device=torch.device("cuda", self.device))}
            self._ctrl_used += nbytes
            self._shapes[key] = st
        st["seq"] += 1
        return st

    # -- buffers
    def x_buffer(self, rows: int, k: int):
        """The peer-readable buffer for this rank's rows — its own slot of the gathered operand: a producer that
        writes its output here hands it to the fused all-gather with no copy at all."""
        from ..ops import native
        if rows > self.max_rows or k > self.max_k:
            raise ValueError(f"rows x k = {rows} x {k} exceeds the workspace ({self.max_rows} x {self.max_k})")
        return native().tensor_from_ptr(self.base + self.off_gathered + self.rank * rows * k * 2, [rows, k], "bf16", self.device)

    def last_gathered(self, rows: int, k: int):
        """The (world * rows, k) operand the last ``ag_gemm`` assembled (valid until the next one): the weight
        gradient of a column-parallel linear needs exactly this matrix."""
        if self.lane != "p2p":
            return self._last_full
        from ..ops import native
        return native().tensor_from_ptr(self.base + self.off_gathered, [rows * self.world, k], "bf16", self.device)

    def all_gather(self, x, full=None):
        """(rows, k) -> (world * rows, k), no GEMM attached (operands of weight gradients in the backward).  With ``full``
        given this is the group ABI's form: every rank's ``x`` lands in ``full``, rank order."""
        import torch
        import torch.distributed as dist
        if full is not None:
            return GroupCollectives.all_gather(self, x, full)
        out = torch.empty(x.shape[0] * self.world, x.shape[1], dtype=x.dtype, device=x.device)
        if self.world == 1:
            out.copy_(x)
        else:
            dist.all_gather_into_tensor(out, x.contiguous(), group=self.pg)
        return out

    def all_reduce(self, t, op: str = "sum"):
        import torch.distributed as dist
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM, group=self.pg)
        return t

    # -- fused ops
    def ag_gemm(self, x, w, out=None, w_is_kn: bool = True):
        """``x``: this rank's rows (rows, K) — ideally ``x_buffer`` itself; ``w``: (K, N) when ``w_is_kn`` else (N, K).
        Returns (world * rows, N)."""
        import torch
        rows, k = x.shape
        n = w.shape[1] if w_is_kn else w.shape[0]
        if out is None:
            out = torch.empty(rows * self.world, n, dtype=x.dtype, device=x.device)
        if self.lane != "p2p":
            import torch.distributed as dist
            parts = [torch.empty_like(x) for _ in range(self.world)]
            dist.all_gather(parts, x.contiguous(), group=self.pg)
            full = torch.cat(parts, 0)
            self._last_full = full
            out.copy_(torch.matmul(full.float(), (w if w_is_kn else w.t()).float()).to(out.dtype))
            return out
        from ..ops import native
        from ..ops.cuda import LAUNCHES
        xb = self.x_buffer(rows, k)
        if x.data_ptr() != xb.data_ptr():
            xb.copy_(x)
        st = self._words(("ag", rows, k), 32)
        chunk = 16 if rows % 16 == 0 else rows
        slot = rows * k * 2
        native().tp_ag_gemm([p + self.off_gathered + r * slot for r, p in enumerate(self.ws)], k, self.base + self.off_gathered,
                            w, w_is_kn, out, rows, self.rank,
                            st["flags"], [p + st["off"] for p in self.ws], [p + st["off"] + 64 for p in self.ws], st["seq"],
                            chunk, self.timeout_s, self.err, self.done)
        LAUNCHES.total += 1
        return out

    def gemm_rs(self, x, w, out=None, addend=None, w_is_kn: bool = True):
        """``x``: (world * rows, K) activations; ``w``: this rank's (K, N) shard.  Returns this rank's rows (rows, N) of the
        sum over ranks (+ ``addend``)."""
        import torch
        m, k = x.shape
        rows = m // self.world
        n = w.shape[1] if w_is_kn else w.shape[0]
        if out is None:
            out = torch.empty(rows, n, dtype=x.dtype, device=x.device)
        if self.lane != "p2p":
            import torch.distributed as dist
            part = torch.matmul(x.float(), (w if w_is_kn else w.t()).float())
            if dist.get_backend() == "gloo":
                dist.all_reduce(part, group=self.pg)
                mine = part[self.rank * rows:(self.rank + 1) * rows]
            else:
                mine = torch.empty(rows, n, dtype=torch.float32, device=x.device)
                dist.reduce_scatter_tensor(mine, part, group=self.pg)
            if addend is not None:
                mine = mine + addend.float()
            out.copy_(mine.to(out.dtype))
            return out
        from ..ops import native
        from ..ops.cuda import LAUNCHES
        if rows > self.max_rows or n > self.max_n:
            raise ValueError(f"rows x n = {rows} x {n} exceeds the workspace ({self.max_rows} x {self.max_n})")
        st = self._words(("rs", rows, n), (rows // 256) * ((n + 255) // 256))
        native().tp_gemm_rs(x, w, w_is_kn, out, addend, rows, self.rank, [p + self.off_stage for p in self.ws],
                            [p + st["off"] for p in self.ws], st["seq"], self.timeout_s, self.err, self.done)
        LAUNCHES.total += 1
        return out


def _up(n: int, a: int = 1 << 12) -> int:
    return (int(n) + a - 1) // a * a
