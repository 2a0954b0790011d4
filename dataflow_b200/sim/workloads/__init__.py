"""Analytic workloads: hardware-free programs, their compiler to simulator chains, a model library and summaries."""
from .builders import (MODEL_LIBRARY, AttnSpec, DTypePolicy, LayerSpec, MlpSpec, ModelSpec, ParallelismConfig, TrainingBuilder,
                       TrainingConfig, get_model, trace_training_model)
from .hardware import HARDWARE_PRESETS, HardwareSpec, get_hardware
from .schema import (SCHEMA, SubOp, WorkloadCost, WorkloadObject, WorkloadOutput, WorkloadProgram, WorkloadTask, cost_breakdown,
                     preview_workload, realize_workload, resolve_cost)
from .summary import compute_summary

__all__ = ["MODEL_LIBRARY", "AttnSpec", "DTypePolicy", "LayerSpec", "MlpSpec", "ModelSpec", "ParallelismConfig", "TrainingBuilder",
           "TrainingConfig", "get_model", "trace_training_model", "HARDWARE_PRESETS", "HardwareSpec", "get_hardware", "SCHEMA",
           "SubOp", "WorkloadCost", "WorkloadObject", "WorkloadOutput", "WorkloadProgram", "WorkloadTask", "cost_breakdown",
           "preview_workload", "realize_workload", "resolve_cost", "compute_summary"]
