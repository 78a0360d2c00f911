"""Analytic FLOP / arithmetic-intensity model and the stage-by-stage memory profiler."""
from .flops import calculate_flops_per_token, calculate_arithmetic_intensity, hybrid_flops_per_token, model_flops_utilisation
