"""Evaluation, run comparison and learning-curve plots."""

from ajllm_b200.evaluation.comparison import compare_runs, load_run_summary, write_comparison_csv
from ajllm_b200.evaluation.evaluator import evaluate_model
from ajllm_b200.evaluation.plotting import plot_learning_curves

__all__ = ["compare_runs", "load_run_summary", "write_comparison_csv", "evaluate_model", "plot_learning_curves"]
