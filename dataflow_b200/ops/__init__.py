"""Kernels: hand-written sm_100a CUDA (``cuda``), vendor-library baseline (``library``)
and the pure-PyTorch oracle (``eager``), behind one registry."""
from __future__ import annotations

import os

_mod = None
_load_error: Exception | None = None


def _load():
    global _mod, _load_error
    if _mod is not None or _load_error is not None:
        return _mod
    try:
        import importlib
        import torch  # noqa: F401  (libtorch must be loaded before the extension)
        _mod = importlib.import_module(__name__ + "._ops")
        # device buffers of the engine become tensors through the extension's ``at::from_blob`` from now on
        from ..runtime import interop
        interop.register_device_view_factory(_mod.tensor_from_ptr)
    except Exception as e:  # missing build or missing CUDA libs
        _load_error = e
    return _mod


def native_available() -> bool:
    return _load() is not None


def native():
    """The compiled extension; raises with the build hint if it is missing."""
    mod = _load()
    if mod is None:
        raise RuntimeError("dataflow_b200.ops._ops is not built or failed to load "
                           f"({_load_error!r}); run `python -m dataflow_b200.build`")
    return mod


from .registry import (KernelCtx, KernelImpl, KernelSet, Workspace, device_caps, register,  # noqa: E402
                       registered_ops, resolve_kernels)
