"""Runnable examples: ``python -m llumnix_kv_b200.examples.pd_demo``."""
