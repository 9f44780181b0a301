"""Benchmark drivers (`python -m benchmarks.kvbench ...`, `python benchmarks/<name>.py`)."""
