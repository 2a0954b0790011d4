"""Simulator + planners (CPU only)."""
from .schema import (Event, EventLog, MemoryTracePoint, Object, OutputAlloc, Task, TaskChain,
                     TaskInterval, TransferTrigger)
from .errors import SimulationCapacityError, SimulationError
from .simulator import Simulator, compute_lower_bound, run
from .validate import ValidationError, validate_chain, validate_planning_input
from .stall_report import StallReport, build_stall_report
from .reference_stream import Reference, compute_reference_stream, next_ref_time
