"""Utilities: profiling ranges, validators, balancing helpers, metrics."""
