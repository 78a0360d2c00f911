"""Kernel micro-benchmarks and end-to-end kernel validation (CUDA-event timed)."""
