"""ctypes binding of libnccl: exactly the entry points the daemon lane uses.  The library is the one bundled with
torch (``nvidia/nccl/lib/libnccl.so.2``) or the system one.  No NCCL header is needed: the unique id is an
opaque 128-byte blob, communicators and streams are pointers.
Role parity: reference ``src/dataflow/service/peer/nccl.py:39-209``."""
from __future__ import annotations

import ctypes
import glob
import os

NCCL_UNIQUE_ID_BYTES = 128
DTYPES = {"int8": 0, "uint8": 1, "int32": 2, "uint32": 3, "int64": 4, "uint64": 5, "fp16": 6, "fp32": 7, "fp64": 8, "bf16": 9}
OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}


class NcclError(RuntimeError):
    pass


class UniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * NCCL_UNIQUE_ID_BYTES)]


def find_library() -> str:
    cands = []
    try:
        import nvidia.nccl
        cands += glob.glob(os.path.join(os.path.dirname(nvidia.nccl.__file__), "lib", "libnccl.so*"))
    except Exception:       # noqa: BLE001
        pass
    try:
        import torch
        cands += glob.glob(os.path.join(os.path.dirname(torch.__file__), "lib", "libnccl.so*"))
    except Exception:       # noqa: BLE001
        pass
    cands += ["libnccl.so.2", "libnccl.so"]
    for c in cands:
        try:
            ctypes.CDLL(c)
            return c
        except OSError:
            continue
    raise NcclError("libnccl was not found (looked in the torch / nvidia-nccl packages and the loader path)")


class Lib:
    _instance = None

    def __init__(self, path: str | None = None):
        self.path = path or find_library()
        L = self.lib = ctypes.CDLL(self.path)
        vp, i, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
        L.ncclGetErrorString.restype = ctypes.c_char_p
        L.ncclGetErrorString.argtypes = [i]
        sigs = {
            "ncclGetVersion": [ctypes.POINTER(i)],
            "ncclGetUniqueId": [ctypes.POINTER(UniqueId)],
            "ncclCommInitRank": [ctypes.POINTER(vp), i, UniqueId, i],
            "ncclCommDestroy": [vp], "ncclCommAbort": [vp],
            "ncclCommGetAsyncError": [vp, ctypes.POINTER(i)],
            "ncclAllReduce": [vp, vp, sz, i, i, vp, vp],
            "ncclBroadcast": [vp, vp, sz, i, i, vp, vp],
            "ncclReduce": [vp, vp, sz, i, i, i, vp, vp],
            "ncclReduceScatter": [vp, vp, sz, i, i, vp, vp],
            "ncclAllGather": [vp, vp, sz, i, vp, vp],
            "ncclSend": [vp, sz, i, i, vp, vp], "ncclRecv": [vp, sz, i, i, vp, vp],
            "ncclGroupStart": [], "ncclGroupEnd": [],
        }
        for name, args in sigs.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = i, args

    @classmethod
    def get(cls) -> "Lib":
        if cls._instance is None:
            cls._instance = Lib()
        return cls._instance

    def check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise NcclError(f"{what}: {self.lib.ncclGetErrorString(rc).decode()} (code {rc})")

    def version(self) -> int:
        v = ctypes.c_int()
        self.check(self.lib.ncclGetVersion(ctypes.byref(v)), "ncclGetVersion")
        return v.value

    def unique_id(self) -> bytes:
        uid = UniqueId()
        self.check(self.lib.ncclGetUniqueId(ctypes.byref(uid)), "ncclGetUniqueId")
        return bytes(uid.internal)

    def comm_init_rank(self, world: int, uid: bytes, rank: int) -> ctypes.c_void_p:
        u = UniqueId()
        ctypes.memmove(u.internal, uid, NCCL_UNIQUE_ID_BYTES)
        comm = ctypes.c_void_p()
        self.check(self.lib.ncclCommInitRank(ctypes.byref(comm), world, u, rank), "ncclCommInitRank")
        return comm
