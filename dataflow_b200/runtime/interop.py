"""Zero-copy bridges between engine buffers and torch tensors, and between engine
streams and torch streams.  torch is imported lazily so the runtime package stays
torch-free at import.  Role parity: reference ``src/dataflow/runtime/interop.py:34-197``
(there a hand-built DLPack capsule; here ``at::from_blob`` inside the extension for
device memory and ``torch.frombuffer`` over a ctypes window for host memory).
"""
from __future__ import annotations

import ctypes
from typing import Sequence

TORCH_DTYPE_BY_NAME: dict[str, object] = {}
_ITEMSIZE = {"fp32": 4, "bf16": 2, "fp16": 2, "int32": 4, "int64": 8, "int16": 2, "uint8": 1, "int8": 1, "fp64": 8, "bool": 1,
             "fp8_e4m3": 1, "fp8_e5m2": 1}


def _dtypes():
    if not TORCH_DTYPE_BY_NAME:
        import torch
        TORCH_DTYPE_BY_NAME.update({
            "fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16, "int32": torch.int32,
            "int64": torch.int64, "int16": torch.int16, "uint8": torch.uint8, "int8": torch.int8, "fp64": torch.float64,
            "bool": torch.bool, "fp8_e4m3": torch.float8_e4m3fn, "fp8_e5m2": torch.float8_e5m2})
    return TORCH_DTYPE_BY_NAME


def dtype_name(torch_dtype) -> str:
    for k, v in _dtypes().items():
        if v == torch_dtype:
            return k
    raise KeyError(torch_dtype)


_view_cache: dict[tuple, object] = {}

# How a device address becomes a tensor.  The runtime itself knows one way that needs nothing but torch (the CUDA array
# interface); a package that has a faster native factory (``at::from_blob`` inside an extension) registers it here when it
# is imported.  The runtime never imports such a package itself.
_device_factory = None


def register_device_view_factory(fn) -> None:
    """``fn(address, shape_list, dtype_name, device_ordinal) -> tensor`` aliasing device memory."""
    global _device_factory
    _device_factory = fn


class _DeviceWindow:
    """``nbytes`` of device memory at ``ptr`` through the CUDA array interface (a zero-copy import for torch)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _device_view(ptr: int, shape, dtype: str, nbytes: int, device: int):
    import torch
    if _device_factory is not None:
        return _device_factory(ptr, list(shape), dtype, device)
    if nbytes == 0:
        return torch.empty(shape, dtype=_dtypes()[dtype], device=torch.device("cuda", device))
    raw = torch.as_tensor(_DeviceWindow(ptr, nbytes), device=torch.device("cuda", device))
    return raw.view(_dtypes()[dtype]).reshape(shape)


def torch_view(buffer, shape: Sequence[int], dtype: str = "bf16", offset_bytes: int = 0, device: int | None = None):
    """Tensor aliasing ``buffer`` (an object with ``ptr`` and ``size``, or a raw address).

    ``device``: CUDA ordinal for device memory, ``None`` for host memory (pinned or not).
    Views are cached by (address, shape, dtype, device); call :func:`invalidate_views`
    when the underlying memory is returned to its pool.
    """
    import torch
    ptr = int(getattr(buffer, "ptr", buffer)) + int(offset_bytes)
    shape = tuple(int(s) for s in shape)
    key = (ptr, shape, dtype, device)
    t = _view_cache.get(key)
    if t is not None:
        return t
    n = 1
    for s in shape:
        n *= s
    nbytes = n * _ITEMSIZE[dtype]
    size = getattr(buffer, "size", None)
    if size is not None and offset_bytes + nbytes > size:
        raise ValueError(f"view of {nbytes} bytes at offset {offset_bytes} exceeds the {size}-byte buffer")
    if device is None:
        if nbytes == 0:
            t = torch.empty(shape, dtype=_dtypes()[dtype])
        else:
            window = (ctypes.c_char * nbytes).from_address(ptr)
            t = torch.frombuffer(window, dtype=torch.uint8).view(_dtypes()[dtype]).reshape(shape)
    else:
        t = _device_view(ptr, shape, dtype, nbytes, int(device))
    if len(_view_cache) > 65536:
        _view_cache.clear()
    _view_cache[key] = t
    return t


def invalidate_views() -> None:
    _view_cache.clear()


_stream_cache: dict[int, object] = {}


def external_stream(handle: int, device: int = 0):
    """Wrap a raw ``cudaStream_t`` as a ``torch.cuda.ExternalStream`` (cached)."""
    import torch
    s = _stream_cache.get(handle)
    if s is None:
        s = torch.cuda.ExternalStream(handle, device=device)
        _stream_cache[handle] = s
    return s
