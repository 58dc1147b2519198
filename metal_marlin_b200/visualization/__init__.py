"""Quantization-error analysis and pictures: error metrics of a quantized tensor, an analyzer over layers and formats, a
visualizer that quantizes the matrices of a checkpoint in the formats of this package and reports on them, and the plots
(weight comparison, error distribution, per-layer errors, error heat map) drawn straight into images with Pillow — there is
no plotting library dependency.

Parity: reference ``visualization/__init__.py`` (``WeightVisualizer`` with ``from_safetensors`` / ``compare_quantization`` /
``generate_error_report`` / ``plot_error_heatmap``; ``plot_weight_comparison`` / ``plot_error_distribution`` / ``plot_layer_errors``) and
``visualization/error_analysis.py`` (``ErrorMetrics`` :23 with ``from_tensors`` / ``to_dict``; ``ErrorAnalyzer`` :167 with ``add_layer_metrics`` /
``get_layer_comparison`` / ``get_format_summary`` / ``get_best_format_per_layer`` / ``identify_problematic_layers``).
"""
from .error_analysis import ErrorAnalyzer, ErrorMetrics
from .plots import plot_error_distribution, plot_error_heatmap, plot_layer_errors, plot_weight_comparison
from .visualizer import WeightVisualizer

__all__ = ["WeightVisualizer", "ErrorAnalyzer", "ErrorMetrics", "plot_weight_comparison", "plot_error_distribution", "plot_layer_errors",
           "plot_error_heatmap"]
