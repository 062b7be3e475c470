"""Micro-benchmarks and roofline helpers (device-timed with CUDA events)."""
