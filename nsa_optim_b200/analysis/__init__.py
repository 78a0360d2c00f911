"""Result loading, comparisons, reports and curves for finished runs."""
from .analysis import (ExperimentResult, load_experiment_results, compare_optimizers, compare_attention_types,
                       compare_context_lengths, generate_report, plot_training_curves, evaluate_model)
