"""The stages of the throughput-fidelity study, one module each; ``run_experiment.py`` strings them together."""
