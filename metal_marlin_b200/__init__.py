"""B200-native quantized LLM inference engine: the capabilities, public API and checkpoint formats of metal-marlin on
NVIDIA B200 (sm_100a) - PyTorch for the framework layer, hand-written CUDA kernels (``metal_marlin_b200/_C.so``) for
every hot op, in-kernel NVLink exchange for tensor / expert parallel decode.

Parity: reference ``metal_marlin/__init__.py:19-518`` (package facade re-exporting ~150 names with optional-import
guards).  Names are resolved lazily on first access so importing the package stays cheap and never needs a GPU.
"""
from __future__ import annotations

import importlib
from typing import Dict, Tuple

__version__ = "0.1.0"

# public name -> (module, attribute)
_EXPORTS: Dict[str, Tuple[str, str]] = {}


def _reg(module: str, *names: str, **aliases: str) -> None:
    for n in names:
        _EXPORTS[n] = (module, n)
    for alias, target in aliases.items():
        _EXPORTS[alias] = (module, target)


_reg("._compat", "E2M1_VALUES", "NF4_VALUES")
_reg(".compat_api", "silu_metal", "gelu_metal", "relu_metal", "swiglu_fused_metal", "geglu_fused_metal", "GemmFp4", "GemmInt8", "pack_int8_weights",
     "unpack_int8_weights")
_reg(".memory.pools", "TransientBuffer", "TransientBufferCPP", "get_transient_buffer_cpp", "reset_transient_buffer_cpp", "transient_buffer_cpp_stats")
_reg(".converters.activation_stats", "CalibrationDatasetLoader", "compute_activation_ranges", "ranges_to_scales", "save_ranges", "load_ranges")
_reg(".models.qwen36_profile", "Qwen36ModelProfile", "QWEN36_27B_PROFILE", "profile_from_hf_config", "load_profile_from_config_file",
     "shape_contract_payload", "is_qwen36_27b_profile", "is_qwen36_27b_config", "validate_supported_profile")
_reg(".utils.memory", "pad_to_multiple", "unpad")
_reg(".converters.torch_compat", "export_for_pytorch", "import_from_pytorch")
_reg(".memory.expert_cache", "ExpertWeightStreamer")
_reg(".attention", "BlockSparseMask", "block_sparse_attention_metal")
_reg(".moe.fast_router", "MoERouterCpp", "RouterBatchOutput")
_reg(".trellis.lm", TrellisConfig="TrellisModelConfig")
_reg(".compat_api", "cholesky_decompose", "is_expert_buffer_pool_available", "initialize_expert_buffer_pool", "get_expert_buffer_pool",
     "allocate_expert_weight_buffer", "clear_expert_buffer_pool")
_reg(".analysis.moe_routing", "MoERoutingProfiler", "simulate_routing_for_model", "analyze_routing_from_file")
_reg(".dtypes", "DTypeConfig", "get_dtype_config", "to_torch_dtype")
_reg(".inference.pipeline", "MMFP4Pipeline", "MarlinPipeline", "StreamingOutput")
_reg(".models.mmfp4_causal_lm", MetalMarlinModel="MMFP4ForCausalLM")
_reg(".models.mmfp4_causal_lm", "MMFP4ForCausalLM", "prefill")
_reg(".models.config", "ModelConfig", "get_preset")
_reg(".models.transformer", "Transformer", "PagedKVStorage", "BatchMeta")
_reg(".engine.session", "DecodeSession", "SamplingParams")
_reg(".engine.engine", "LLMEngine")
_reg(".engine.scheduler", "BatchScheduler", "SchedulerConfig", "PreemptionPolicy", "QueueFullError")
_reg(".inference.pipelined", "PipelineScheduler", "AsyncPipelineScheduler", "InferenceRequest", "RequestState", "generate_pipelined")
_reg(".inference.prefill", "PrefillConfig", "PrefillStats", "chunked_prefill", "parallel_kv_write", "flash_prefill_attention",
     "SpeculativePrefillConfig", "speculative_prefill", "pick_chunk_size")
_reg(".inference.decode", "DecodeConfig", "DecodePerfStats", "DecodeState", "persistent_decode_step", "select_decode_kernel",
     "quantized_kv_attention", "quantize_kv_cache")
_reg(".autotune", "KernelAutoTuner", "TunedConfig", "OnlineAdapter", "get_optimal_config")
_reg(".converters.exl3", "detect_exl3_format", "convert_sharded_to_layerwise", "load_exl3_from_hub", "download_exl3_model", "list_exl3_models",
     "parse_model_card", "exl3_layer_to_marlin", "convert_exl3_to_marlin")
_reg(".quant.ldlq", "block_ldl", "ldlq_quantize", "compute_group_scales", "quantize_tile_viterbi", "quantize_tile_greedy", "LDLQResult")
_reg(".engine.fcfs", "FCFSScheduler", "PrefillStrategy", "InsertionPolicy", "CacheInfo")
_reg(".engine.request", "GenerationRequest", "RequestStatus", "RunningRequest", "RequestPriority")
_reg(".sampler", "SamplingConfig", "Sampler", "sample_next_token", MetalSampler="Sampler")
_reg(".rope", "YaRNConfig", "RotaryEmbedding", "apply_rope", "rope_inv_freq", "yarn_inv_freq")
_reg(".kv.contiguous", "KVCache", "KVCacheTorch", "MLAKVCache", "PersistentKVCache", "CacheConfig", "quantize_kv", "dequantize_kv")
_reg(".kv.paged", "BlockAllocator", "MultimodalBlockAllocator", "PageTable", "PrefixCache", "PagedKVCache")
_reg(".layers", "MMFP4Linear", "QuantizedLinear", "TrellisLinear", "HadamardLinear", "Sparse24Linear")
_reg(".ops.weights", "FP4Weight", "FP4ExpertBank")
_reg(".trellis", "TrellisForCausalLM", "TrellisGenerator", "TrellisModelConfig", "GenerationConfig")
_reg(".formats.mmfp4_loader", "MMFP4ModelLoader")
_reg(".formats.trellis", "TrellisModelLoader", "TrellisWeight", "quantize_trellis", "quantize_model_trellis")
_reg(".formats.fp4", "quantize_fp4", "pack_mmfp4", "pack_marlin_fp4", "unpack_mmfp4", "unpack_marlin_fp4")
_reg(".quant.rtn", "quantize", "dequantize", "QuantizedTensor", "pack_bits", "unpack_bits")
_reg(".quant.convert", "convert_model", "convert_model_to_fp4", "convert_model_to_mmfp4", "save_random_checkpoint")
_reg(".quant.gptq", "GPTQConfig", "MRGPTQConfig", "gptq_quantize", "mr_gptq_quantize")
_reg(".quant.awq", "awq_quantize", "awq_search")
_reg(".quant.hadamard", "hadamard_matrix", "block_hadamard", "fwht")
_reg(".quant.calibration", "HessianCollector", "load_calibration_tokens")
_reg(".quant.mixed_precision", "policy_for", "allocate_bits", "TensorPolicy")
_reg(".quant.pipeline", "quantize_checkpoint", "collect_hessians")
_reg(".converters", "convert_checkpoint", "MixedFormatPack")
_reg(".converters.gguf", "GGUFReader", "write_gguf")
_reg(".converters.nemo", "load_nemo")
_reg(".memory.streams", "StreamPool", "EventPool", "AsyncEvent", "discover_devices", "get_stream")
_reg(".quant.psd", "gershgorin_is_psd", "project_psd", "damp_until_cholesky")
_reg(".kv.prompt_cache", "TieredPrefixCache", "RadixPrefixCache", "PrefixCacheConfig", "StorageTier")
_reg(".serving.batching", "RequestBatcher", "BatchConfig", "KVCacheSharing")
_reg(".profiling.wandb_helper", "WandbHelper", "get_wandb")
_reg(".profiling.benchmark_report", "aggregate_results", "generate_markdown_report")
_reg(".inference.early_exit", "EarlyExitModel", "EarlyExitOutput")
_reg(".converters.onnx", "ONNXExecutor", "ONNXGraph", "ONNXOp", "load_onnx", "save_onnx", "parse_onnx_graph", "summarize_graph",
     "detect_architecture")
_reg(".spec.engine", "SpeculativeEngine")
_reg(".spec.draft", "NGramDraft", "SmallModelDraft", "MTPDraft", "MTPHead", "EagleDraft", "DraftModel")
_reg(".spec.verify", "verify_greedy", "verify_speculative", "verify_batch_greedy", "verify_tree_greedy", "tree_attention_mask")
_reg(".spec.adaptive", "AdaptiveSpeculationController", "TokenAcceptanceTracker")
_reg(".serving.engine", "ServingEngine", "EngineConfig")
_reg(".serving.server", "run_server")
_reg(".serving.metrics", "MetricsCollector", "MoEMetrics", "PerplexityTracker")
_reg(".eval", "compute_perplexity", "kl_divergence", "quality_report", "ExpertUsageProfiler", "load_balancing_loss")
_reg(".inference.long_context", "LongContextConfig", "LongContextModel", "StreamingAttention", "chunked_attention", "sliding_window_mask")
_reg(".attention", "block_sparse_attention", "sliding_window_attention", "tree_attention", "differential_attention")
_reg(".arch", "MambaBlock", "MambaConfig", "selective_scan", "gated_delta_rule_chunked", "gated_delta_step", "wkv5", "wkv6", "layout_from_config")
_reg(".vision", "ImagePreprocessor", "PreprocessConfig", "LlavaProjector", "PatchMergerProjector", "VisionEncoderCache")
_reg(".hf", "replace_linear_layers", "find_linear_layers", "find_moe_layers", "load_prequantized_mmfp4_model", "replace_moe_layers",
     "replace_moe_layers_streaming", "quantize_moe_experts", "QuantizedMoEExperts", "QuantizedMoEBlock")
_reg(".memory", "Arena", "BumpAllocator", "WorkspaceBuffer", "ExpertCache", "PinnedPool", "WeightStreamer", "MemoryPressureMonitor")
_reg(".parallel.tp", "TPContext", "shard_transformer", "make_context")
_reg(".parallel.mesh", "DeviceMesh", "MeshShape", "plan_mesh")
_reg(".parallel.ep", "ExpertParallelMoE", "EPExchange")
_reg(".parallel.pp", "PipelineStage", "pipeline_prefill")
_reg(".parallel.cp", "ring_attention")
_reg(".parallel.symm", "SymmetricBuffer")
_reg(".profiling", "KernelTimer", "RooflinePoint", "load_peaks", "trace_scope", "write_trace", "launch_tracer", "profile_kernel")
_reg(".utils", "NaNGuard", "LazyCheckpoint", "load_checkpoint", "save_checkpoint", "remap_weight_keys", "filter_weights")
_reg(".baseline_eager", "EagerBF16Model")


# the reference facade's remaining names (packers, FP8 / Hadamard helpers, MoE dispatch bookkeeping, GEMM / attention entry points,
# RoPE helpers, precision configs, ONNX / vision helpers, memory and dispatch objects) on this engine
_reg(".compat_api",
     "AWQResult", "AdaptiveQuantResult", "AdaptiveQuantizer", "AsyncTransferHandle", "AsyncTransferManager",
     "BatchDispatchContext", "CacheConfigTorch", "CppDispatchInfo", "ExpertManagerCpp", "FP4GPTQQuantizer",
     "FP4Metal", "FP8_E4M3_MAX", "FP8_E4M3_VALUES", "FP8_E5M2_MAX", "FP8_E5M2_VALUES", "FastInferenceContext",
     "GPTQMetal", "GPTQQuantizer", "HAS_MPS", "HAS_PYOBJC_METAL", "HadamardMetadata", "HadamardMetal", "HeapAllocation",
     "HeapAllocatorMetrics", "HeapBufferPool", "HessianManager", "InternVLProjector", "LLaVAProjector", "LayerBudget",
     "LayerPrecisionSelector", "LayerQuantConfig", "LayerSensitivity", "MLAAttentionCpp", "MRGPTQQuantizer",
     "MarlinAttention", "MarlinLinear", "MetalHeapAllocator", "MetalQuantizedLinear", "MetalQuantizedMoE", "MixedPrecisionConfig",
     "MoEDispatchInfo", "MoEPrecisionConfig", "ModelBudgetAllocation", "ONNXGraphInfo", "PipelinedLayerDispatcher",
     "Precision", "QuantizationFormat", "QuantizationReport", "Qwen2VLProjector", "RoPE", "VisionProjector",
     "VisionProjectorConfig", "YaRNRoPE", "apply_hadamard_rotation", "awq_dequantize", "awq_quantize_model",
     "compute_activation_stats", "compute_expert_load", "compute_fp8_e4m3_values", "compute_fp8_e5m2_values",
     "compute_hessian_metal", "compute_load_balancing_loss", "compute_moe_expert_sensitivity", "compute_salient_scaling",
     "compute_yarn_cos_sin_cache", "compute_yarn_inv_freq", "create_causal_mask", "create_expert_manager", "create_rope_from_config",
     "create_sliding_window_mask", "dequant_fp8_e4m3", "dequant_fp8_e5m2", "dequantize_fp4_metal", "dequantize_fp8_e4m3",
     "dequantize_fp8_e5m2", "dequantize_kv_cache_fp8", "dequantize_kv_cache_fp8_e5m2", "dequantize_mmfp4", "detect_projector_type",
     "dispatch_batched_gemm_variable_seq", "dispatch_grouped_attention_variable_seq", "expert_gather", "expert_manager_available",
     "expert_scatter_add", "extract_onnx_weights", "fast_dispatch_available", "find_salient_weights", "flash_attention_metal",
     "fused_moe_forward", "gather_for_experts", "generate", "generate_batch", "generate_stream", "get_fast_context",
     "get_onnx_config", "get_parent_module", "get_yarn_mscale", "group_tokens_by_expert", "group_tokens_by_expert_full",
     "hadamard_transform_metal", "inverse_hadamard_rotation", "list_onnx_tensors", "marlin_gemm_fp4", "marlin_gemm_int4",
     "mla_cpp_available", "mmfp4_fused_qkv", "mmfp4_gemm", "normalize_onnx_name", "pack_fp4_weights", "pack_fp4_weights_cpu",
     "pack_fp8_weights", "pack_int4_weights", "pack_nf4_weights", "parse_onnx_graph_full", "quantize_fp4_metal",
     "quantize_kv_cache_fp8", "quantize_kv_cache_fp8_e5m2", "quantize_linear_layer", "quantize_to_fp8", "quantize_to_fp8_e4m3",
     "quantize_to_fp8_e5m2", "quantize_to_int4", "quantize_to_nf4", "scaled_dot_product_attention_metal", "scatter_expert_outputs",
     "sliding_window_attention_metal", "unpack_fp4_weights")


def __getattr__(name: str):
    try:
        module, attr = _EXPORTS[name]
    except KeyError:
        raise AttributeError(f"module 'metal_marlin_b200' has no attribute {name!r}") from None
    val = getattr(importlib.import_module(module, __name__), attr)
    globals()[name] = val
    return val


def __dir__():
    return sorted(list(globals()) + list(_EXPORTS))


def has_cuda_kernels() -> bool:
    """True when a GPU is present and the native library is loaded (the CUDA path is the one that will run)."""
    from . import ops
    return ops.native_available()


HAS_TORCH = True
__all__ = sorted(_EXPORTS) + ["__version__", "has_cuda_kernels", "HAS_TORCH"]
