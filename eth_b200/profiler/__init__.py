"""Profiler: CUDA-event micro-benchmarks of ops, collectives and P2P, writing the profile schema."""
