from .moe_routing import ExpertUsageProfiler, apply_capacity, load_balancing_loss
from .perplexity import compute_perplexity, kl_divergence, quality_report, sliding_window_nll, synthetic_corpus

__all__ = ["ExpertUsageProfiler", "apply_capacity", "load_balancing_loss", "compute_perplexity", "kl_divergence", "quality_report",
           "sliding_window_nll", "synthetic_corpus"]
