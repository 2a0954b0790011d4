"""dataflow_b200 — a B200-native memory-constrained training runtime.

A model + training config is lowered to a *Dataflow Program* (``core``), planned
against a fast-memory budget by a simulator-verified planner (``sim``), and run
by a native task executor (``runtime``) whose hot ops are hand-written sm_100a
kernels (``ops``), with collectives fused over NVLink peer memory (``parallel``).
"""
__version__ = "0.1.0"


def code_revision() -> str:
    """A digest of this package's source files (Python, CUDA, C++): what two processes must agree on before they run one job
    together.  ``DATAFLOW_CODE_REV`` overrides it (tests)."""
    import hashlib
    import os
    forced = os.environ.get("DATAFLOW_CODE_REV")
    if forced:
        return forced
    global _CODE_REV
    if _CODE_REV is None:
        root = os.path.dirname(os.path.abspath(__file__))
        h = hashlib.sha256()
        for d, dirs, files in sorted(os.walk(root)):
            dirs[:] = sorted(x for x in dirs if x not in ("__pycache__", "build"))
            for f in sorted(files):
                if f.endswith((".py", ".cu", ".cuh", ".cpp", ".hpp", ".h")):
                    path = os.path.join(d, f)
                    h.update(os.path.relpath(path, root).encode())
                    with open(path, "rb") as fh:
                        h.update(fh.read())
        _CODE_REV = h.hexdigest()[:16]
    return _CODE_REV


_CODE_REV = None


def environment_line() -> str:
    """What replicated compute must share besides the code: the framework and CUDA versions (another version may pick other
    kernels, and replicas then drift apart silently)."""
    try:
        import torch
        return f"torch {torch.__version__} cuda {torch.version.cuda}"
    except Exception:       # noqa: BLE001
        return "torch absent"
