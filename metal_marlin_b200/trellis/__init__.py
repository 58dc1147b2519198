"""Trellis stack: causal LM and generator on the shared decoder, plus building blocks, packing / dispatch functions and the
mixed-bit auto-tuner under the reference's ``metal_marlin.trellis`` names."""
from .generate import GenerationConfig, TrellisGenerator
from .layers import (GLM4_TOKENIZER_ID, CausalLMOutput, CompressedKVCache, MixedBPWMoEDispatcher, MoEConfig, TrellisDecoderLayer,
                     TrellisDenseMLP, TrellisExpert, TrellisKVCache, TrellisMLAConfig, TrellisMLAttention, TrellisMoELayer, TrellisMoEMLP,
                     compute_compression_ratio, compute_packed_size, create_mla_projections, dequantize_trellis_weight,
                     dispatch_gemm_trellis_auto, dispatch_gemm_trellis_decode_auto, dispatch_mixed_bpw_moe,
                     dispatch_mixed_bpw_moe_with_cpp_fallback, dispatch_sign_flips, dispatch_trellis_dequant,
                     dispatch_trellis_dequant_fused, dispatch_trellis_dequant_packed, get_mixed_bpw_stats, pack_indices,
                     pack_indices_vectorized, pack_trellis_indices, reset_mixed_bpw_stats, unpack_indices, unpack_indices_vectorized,
                     unpack_trellis_indices)
from .lm import TrellisForCausalLM, TrellisModelConfig
from ..layers.linear import TrellisLinear

TrellisModelWrapper = TrellisForCausalLM


def __getattr__(name: str):
    if name in ("MixedKernelSelector", "KernelABTester", "KernelFeedback", "ExpertSelectionCache", "ExpertMemoryPool", "select_intelligent_kernel",
                "get_kernel_for_batch_size"):
        from . import kernel_selection
        return getattr(kernel_selection, name)
    if name in ("create_mock_trellis_linear", "create_mock_dense_mlp", "create_mock_moe_mlp", "create_mini_config", "create_mini_model"):
        from . import testing
        return getattr(testing, name)
    if name in ("TrellisWeight", "TrellisModelLoader"):
        from ..formats import trellis as fmt
        return getattr(fmt, name)
    if name in ("MixedBPWAutoTuner", "AutotuneConfig", "KernelConfig", "BenchmarkResult", "TrellisModel"):
        if name == "TrellisModel":                      # the decoder under the wrapper
            from ..models.transformer import Transformer
            return Transformer
        from .. import autotune as at
        return {"MixedBPWAutoTuner": at.KernelAutoTuner, "AutotuneConfig": at.TunedConfig, "KernelConfig": at.TunedConfig,
                "BenchmarkResult": dict}[name]
    raise AttributeError(name)


__all__ = ["MixedKernelSelector", "KernelABTester", "KernelFeedback", "ExpertSelectionCache", "ExpertMemoryPool", "select_intelligent_kernel",
           "get_kernel_for_batch_size", "create_mock_trellis_linear", "create_mock_dense_mlp", "create_mock_moe_mlp", "create_mini_config",
           "create_mini_model", "TrellisWeight", "TrellisModelLoader", "GenerationConfig", "TrellisGenerator", "TrellisForCausalLM", "TrellisModelConfig", "TrellisLinear", "TrellisModelWrapper",
           "TrellisModel", "MixedBPWAutoTuner", "AutotuneConfig", "KernelConfig", "BenchmarkResult", "GLM4_TOKENIZER_ID", "CausalLMOutput",
           "CompressedKVCache", "MixedBPWMoEDispatcher", "MoEConfig", "TrellisDecoderLayer", "TrellisDenseMLP", "TrellisExpert",
           "TrellisKVCache", "TrellisMLAConfig", "TrellisMLAttention", "TrellisMoELayer", "TrellisMoEMLP", "compute_compression_ratio",
           "compute_packed_size", "create_mla_projections", "dequantize_trellis_weight", "dispatch_gemm_trellis_auto",
           "dispatch_gemm_trellis_decode_auto", "dispatch_mixed_bpw_moe", "dispatch_mixed_bpw_moe_with_cpp_fallback", "dispatch_sign_flips",
           "dispatch_trellis_dequant", "dispatch_trellis_dequant_fused", "dispatch_trellis_dequant_packed", "get_mixed_bpw_stats",
           "pack_indices", "pack_indices_vectorized", "pack_trellis_indices", "reset_mixed_bpw_stats", "unpack_indices",
           "unpack_indices_vectorized", "unpack_trellis_indices"]
