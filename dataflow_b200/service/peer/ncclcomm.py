"""A peer group on NCCL: the communicator is built from a unique id the coordinator broadcasts over the control
star (it rides the GROUP_JOIN frame), collectives run on a private stream with explicit event edges to the caller's
stream, and an asynchronous error aborts the communicator instead of hanging the daemon.
Role parity: reference ``src/dataflow/service/peer/ncclcomm.py:26-127``."""
from __future__ import annotations

import ctypes

from .nccl import DTYPES, OPS, Lib, NcclError

_TORCH_DTYPE = {"torch.float32": "fp32", "torch.bfloat16": "bf16", "torch.float16": "fp16", "torch.int32": "int32",
                "torch.int64": "int64", "torch.uint8": "uint8", "torch.int8": "int8", "torch.float64": "fp64"}


class NcclComm:
    def __init__(self, name: str, rank: int, world: int, uid: bytes, device: int):
        import torch
        self.name, self.rank, self.world, self.device = name, rank, world, device
        self.lib = Lib.get()
        torch.cuda.set_device(device)
        self.comm = self.lib.comm_init_rank(world, uid, rank)
        self.stream = torch.cuda.Stream(device=device)
        self.failed = ""

    @staticmethod
    def new_unique_id() -> bytes:
        return Lib.get().unique_id()

    def _edges(self):
        import contextlib
        import torch

        @contextlib.contextmanager
        def scope():
            cur = torch.cuda.current_stream(self.device)
            e0 = torch.cuda.Event()
            e0.record(cur)
            self.stream.wait_event(e0)
            yield ctypes.c_void_p(self.stream.cuda_stream)
            e1 = torch.cuda.Event()
            e1.record(self.stream)
            cur.wait_event(e1)
        return scope()

    def _dt(self, t) -> int:
        return DTYPES[_TORCH_DTYPE[str(t.dtype)]]

    def guard(self) -> None:
        """Raise (and abort the communicator) if NCCL reported an asynchronous error."""
        if self.failed:
            raise NcclError(f"group {self.name}: {self.failed}")
        err = ctypes.c_int()
        self.lib.check(self.lib.lib.ncclCommGetAsyncError(self.comm, ctypes.byref(err)), "ncclCommGetAsyncError")
        if err.value != 0:
            self.fail(f"asynchronous NCCL error {err.value}")
            raise NcclError(f"group {self.name}: {self.failed}")

    def all_reduce(self, t, op: str = "sum"):
        self.guard()
        with self._edges() as s:
            self.lib.check(self.lib.lib.ncclAllReduce(t.data_ptr(), t.data_ptr(), t.numel(), self._dt(t), OPS[op], self.comm, s), "ncclAllReduce")
        return t

    def reduce_scatter(self, out, inp, op: str = "sum"):
        self.guard()
        with self._edges() as s:
            self.lib.check(self.lib.lib.ncclReduceScatter(inp.data_ptr(), out.data_ptr(), out.numel(), self._dt(inp), OPS[op], self.comm, s),
                           "ncclReduceScatter")
        return out

    def all_gather(self, out, inp):
        self.guard()
        with self._edges() as s:
            self.lib.check(self.lib.lib.ncclAllGather(inp.data_ptr(), out.data_ptr(), inp.numel(), self._dt(inp), self.comm, s), "ncclAllGather")
        return out

    def broadcast(self, t, root: int = 0):
        self.guard()
        with self._edges() as s:
            self.lib.check(self.lib.lib.ncclBroadcast(t.data_ptr(), t.data_ptr(), t.numel(), self._dt(t), root, self.comm, s), "ncclBroadcast")
        return t

    def reduce(self, t, root: int = 0, op: str = "sum"):
        """Sum lands in ``root``'s tensor; the other ranks' tensors keep their values (reduced into a scratch copy there)."""
        self.guard()
        dst = t if self.rank == root else t.clone()
        with self._edges() as s:
            self.lib.check(self.lib.lib.ncclReduce(t.data_ptr(), dst.data_ptr(), t.numel(), self._dt(t), OPS[op], root,
                                                   self.comm, s), "ncclReduce")
        return t

    def send(self, t, peer: int):
        """Point-to-point (pipeline stages): stays on NCCL, overlapped on the group's stream."""
        self.guard()
        with self._edges() as s:
            self.lib.check(self.lib.lib.ncclSend(t.data_ptr(), t.numel(), self._dt(t), peer, self.comm, s), "ncclSend")

    def recv(self, t, peer: int):
        self.guard()
        with self._edges() as s:
            self.lib.check(self.lib.lib.ncclRecv(t.data_ptr(), t.numel(), self._dt(t), peer, self.comm, s), "ncclRecv")
        return t

    def warm_up(self) -> None:
        import torch
        x = torch.ones(1, device=torch.device("cuda", self.device))
        self.all_reduce(x)
        torch.cuda.synchronize(self.device)
        if float(x) != float(self.world):
            self.fail(f"warm-up all-reduce returned {float(x)} for world {self.world}")
            raise NcclError(self.failed)

    def fail(self, why: str) -> None:
        if not self.failed:
            self.failed = why
            if self.comm:
                self.lib.lib.ncclCommAbort(self.comm)
                self.comm = None

    def close(self) -> None:
        if self.comm:
            self.lib.lib.ncclCommDestroy(self.comm)
            self.comm = None
