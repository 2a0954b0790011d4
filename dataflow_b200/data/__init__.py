"""Data plane: sources -> feed -> packer -> per-round int32 buffers + segment bounds (see ``pipeline``)."""
from .sequence import IGNORE_INDEX, PackedRound, PackedStep, Sequence
from .feed import DataFeed
from .packer import Packer
from .pipeline import DataPipeline, PrepackedPipeline, fast_forward, legacy_block_pipeline, pipeline_from_args
from .sources import DataSource, resolve_data
from .segments import Segments
