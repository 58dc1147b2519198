"""Utilities: checkpoint IO, NaN guard, canary buffers, FLOP calculators, memory queries / padding / prefetching and
call-level profiling (the reference's ``metal_marlin.utils`` surface)."""
from .checkpoint import LazyCheckpoint, filter_weights, load_checkpoint, load_sharded_checkpoint, remap_weight_keys, save_checkpoint
from .flops_calculator import (LayerFLOPsCalculator, LayerProfileConfig, ModuleFLOPsResult, calculate_layer_flops, estimate_marlin_linear_flops,
                               profile_model_layers)
from .memory import (AdaptivePrefetcher, MemoryInfo, SystemMemoryInfo, TensorMetadata, compute_optimal_batch_size,
                     estimate_tensor_memory, get_metal_memory_pressure, get_system_memory, get_system_memory_detailed, pad_numpy_2d,
                     pad_to_multiple, pad_torch_2d, round_up, should_reduce_allocation, unpad)
from .nan_guard import NaNGuard, NaNStats
from .profile_ops import (LayerFLOPs, LayerFLOPsCounter, TransformerLayerFLOPs, calculate_attention_flops, calculate_embedding_flops,
                          calculate_ffn_flops, calculate_layernorm_flops, calculate_matmul_flops, profile_model_flops)
from .profiling import (ProfileRecord, ProfileStats, clear_profiles, disable_profiling, enable_profiling, get_all_profile_stats,
                        get_profile_records, get_profile_stats, is_profiling_enabled, print_profile_summary, profile_kernel)

__all__ = ["LazyCheckpoint", "filter_weights", "load_checkpoint", "load_sharded_checkpoint", "remap_weight_keys", "save_checkpoint", "NaNGuard",
           "NaNStats", "AdaptivePrefetcher", "MemoryInfo", "SystemMemoryInfo", "TensorMetadata", "compute_optimal_batch_size",
           "estimate_tensor_memory", "get_metal_memory_pressure", "get_system_memory", "get_system_memory_detailed", "pad_numpy_2d",
           "pad_torch_2d", "round_up", "should_reduce_allocation", "pad_to_multiple", "unpad", "LayerFLOPs", "LayerFLOPsCounter", "TransformerLayerFLOPs",
           "calculate_attention_flops", "calculate_embedding_flops", "calculate_ffn_flops", "calculate_layernorm_flops",
           "calculate_matmul_flops", "profile_model_flops", "ProfileRecord", "ProfileStats", "clear_profiles", "disable_profiling",
           "enable_profiling", "get_all_profile_stats", "get_profile_records", "get_profile_stats", "is_profiling_enabled",
           "print_profile_summary", "profile_kernel", "LayerFLOPsCalculator", "LayerProfileConfig", "ModuleFLOPsResult", "calculate_layer_flops",
           "estimate_marlin_linear_flops", "profile_model_layers"]


def __getattr__(name: str):
    if name == "TracedDecoderLayer":                 # whole-layer graph capture (reference ``traced`` package)
        from ..engine.traced import TracedDecoderLayer
        return TracedDecoderLayer
    raise AttributeError(name)
