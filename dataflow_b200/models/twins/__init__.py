"""Pure-PyTorch twins: one plain ``nn.Module`` per family, deliberately unoptimised, used as the
correctness oracle for engine runs (role of the reference's ``reference_models/`` tree)."""
