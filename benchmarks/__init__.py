"""Benchmark workloads driven by ``bench.py`` (not part of the installable package)."""
