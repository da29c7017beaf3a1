"""Measurement helpers: seeded synthetic workloads with the shapes of the benchmark configurations
and a CUDA-event timer with L2 flushing (the method of the reference's bench/regime.py:106-136)."""
