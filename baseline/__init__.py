"""Reference arm of the benchmark (see reference_bench.py)."""
