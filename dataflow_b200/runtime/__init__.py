"""Generic execution engine: runs an annotated Program over a device backend.
Workload-agnostic and torch-free (``interop`` imports torch lazily)."""
from . import _runtime
from ._runtime import CpuBackend, FakeBackend, SlabAllocator
from .engine import (ENGINE_INVARIANT_ERRORS, ChainIndex, DeadlockError, Engine, ExecutionError,
                     RunOutcome, RunOutcomeKind, RunResult, Session)
from .executable import (Buffer, Executable, SyntheticExecutable, TaskContext, synthetic_resolver)
from .trace import Interval, RunTrace, compare_to_sim_eventlog, trace_from_dict, trace_to_dict

CudaBackend = getattr(_runtime, "CudaBackend", None)
PoolProbe = getattr(_runtime, "PoolProbe", None)


def set_nvtx(on: bool) -> None:
    """Turn NVTX ranges around tasks and transfers on or off (profiler control)."""
    from . import _runtime
    _runtime.set_nvtx(bool(on))
