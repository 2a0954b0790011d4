"""Lowering: model config → bare Program → planned Program."""
from .shaped_program import (HW_PRESETS, LayerKindSpec, LooseCosts, ShapedConfig, ShapedHardware,
                             build_shaped_program, optimizer_cost_seed, resolve_hardware)
from .planning import DEFAULT_PROGRAM_LEEWAY_BYTES, PlannedProgram, plan_program, strip_plan_annotations, transfer_summary
