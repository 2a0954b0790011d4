"""dataflow_b200 — a B200-native memory-constrained training runtime.

A model + training config is lowered to a *Dataflow Program* (``core``), planned
against a fast-memory budget by a simulator-verified planner (``sim``), and run
by a native task executor (``runtime``) whose hot ops are hand-written sm_100a
kernels (``ops``), with collectives fused over NVLink peer memory (``parallel``).
"""
__version__ = "0.1.0"
