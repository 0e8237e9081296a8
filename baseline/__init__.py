"""Harness that runs the unmodified reference (installed under ``baseline/_ref``)
on the benchmark configs.  Nothing here imports ``flextrain_b200``."""
