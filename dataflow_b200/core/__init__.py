"""Core IR (stdlib only): the Program schema every other layer speaks."""
from .types import (DTYPE_BITS, LOCATIONS, ROLES, Location, Role, TensorMeta, dtype_nbytes)
from .program import (SCHEMA_VERSION, ObjectSpec, OutputSpec, Program, RecomputeOption,
                      RecomputeRewrite, TaskSpec, TransferDirective)
from .validate import ValidationError, collect_problems, validate_program
from .jsonio import (canonical_json, load_program, program_content_id, program_from_dict,
                     program_to_dict, save_program)
from .convert import (apply_chain_annotations, from_sim_chain, to_sim_chain, to_webapp_program)

__all__ = [n for n in dir() if not n.startswith("_")]
