"""Model analysis: the MoE routing profiler (reference ``metal_marlin/analysis``)."""
from .moe_routing import (ExpertCooccurrence, ExpertLoadStats, LayerRoutingProfile, MoERoutingProfiler, RoutingPredictability,
                          analyze_routing_from_file, profile_model, simulate_routing_for_model)

__all__ = ["MoERoutingProfiler", "LayerRoutingProfile", "ExpertLoadStats", "ExpertCooccurrence", "RoutingPredictability", "analyze_routing_from_file",
           "simulate_routing_for_model", "profile_model"]
