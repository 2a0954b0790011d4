"""Policy-gradient fine-tuning on the engine: program surgery on any family's lowering (see ``builder.py``)."""
