"""Checkpoint record layer: the cross-source record, its validation, and restore-plan resolution."""
from .record import (RECORD_FILE, RECORD_SCHEMA, RecordError, build_record, has_record, read_record, validate_record,
                     write_record)
from .targets import persisted_objects, resolve_targets, source_resident_bytes
from .compose import save_checkpoint
