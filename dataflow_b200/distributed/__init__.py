"""Distribution as data: schemes, shard plans, responsibilities, topology, and the fleet helpers."""
from .parallelism import Axis, ParallelismScheme, SchemeError, scheme_from_flags
from .sharding import (Assignment, Region, ShardPlan, expert_shards, local_experts, rs_eligible, tp_attn_shards,
                       tp_mlp_shards, zero_slices)
from .responsibility import Span, responsibility_map
from .source_policy import SourceWrite, compile_source_policy
from .topology import GroupSpec, HostSpec, Member, Topology, load_topology, local_pair_topology, local_topology
from .group_annotation import annotate_groups
