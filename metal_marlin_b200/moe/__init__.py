"""Mixture-of-experts utilities around the kernels: expert capacity and overflow policies, predictive expert prefetching,
load tracking with the auxiliary balancing loss and gate entropy.  The routed-expert math itself lives in ``ops.moe_forward``
(``csrc/moe_*.cu``, ``csrc/gemm_sm100.cu``) and the routing profiler in ``eval/moe_routing.py``."""
from .capacity import (CapacityAnalyzer, CapacityStats, DynamicCapacity, DynamicCapacityConfig, OverflowInfo, OverflowPolicy,
                       analyze_overflow_rate, apply_overflow_policy, auto_tune_capacity, compute_expert_capacity,
                       count_expert_assignments)
from .load_balancing import ExpertLoadTracker, LoadBalancingConfig, gate_entropy, load_balance_loss
from .prefetch import ExpertPrefetcher, PrefetchConfig, PrefetchStrategy
from .router_int8 import Int8Router, Int8RouterLinear, RouterQuantConfig, measure_quantization_error, quantize_router_weights

__all__ = ["CapacityAnalyzer", "CapacityStats", "DynamicCapacity", "DynamicCapacityConfig", "OverflowInfo", "OverflowPolicy",
           "analyze_overflow_rate", "apply_overflow_policy", "auto_tune_capacity", "compute_expert_capacity", "count_expert_assignments",
           "ExpertLoadTracker", "LoadBalancingConfig", "gate_entropy", "load_balance_loss", "ExpertPrefetcher", "PrefetchConfig",
           "PrefetchStrategy", "Int8Router", "Int8RouterLinear", "RouterQuantConfig", "measure_quantization_error",
           "quantize_router_weights"]
