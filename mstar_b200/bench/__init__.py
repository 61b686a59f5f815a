"""Micro- and component benchmarks (python -m mstar_b200.bench.<name>); the serving benchmark is bench.py at the
repository root."""
