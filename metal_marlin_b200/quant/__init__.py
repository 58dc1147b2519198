"""Quantization: round-to-nearest quantizers and packers, GPTQ / MR-GPTQ, AWQ, LDLQ (EXL3-style), Hadamard rotation, PSD
repair, mixed-precision policies and bit allocation, calibration data and Hessian collection, the offline pipeline - and the
reference's ``quantization`` / ``calibration`` package names (``quant/surface.py``).  Resolved on first use."""
from __future__ import annotations

import importlib

_MODULES = {
    ".rtn": ["QuantizedTensor", "quantize", "dequantize", "quantize_fp4", "quantize_int4", "quantize_int8", "quantize_nf4", "quantize_fp8",
             "pack_bits", "unpack_bits", "quantization_error"],
    ".gptq": ["GPTQConfig", "MRGPTQConfig", "gptq_quantize", "mr_gptq_quantize", "quantize_stacked_experts", "ResumableState", "to_quantized_tensor"],
    ".awq": ["awq_search", "awq_quantize", "awq_plan", "apply_awq_plan"],
    ".ldlq": ["block_ldl", "ldl_reconstruct", "compute_group_scales", "quantize_tile_greedy", "proxy_error", "LDLQResult", "ldlq_quantize"],
    ".hadamard": ["hadamard_matrix", "fwht", "block_hadamard", "rotate_weight", "rotate_hessian", "kurtosis"],
    ".psd": ["gershgorin_is_psd", "min_eigenvalue", "project_psd", "damp_until_cholesky"],
    ".mixed_precision": ["TensorPolicy", "policy_for", "allocate_bits"],
    ".calibration": ["HessianCollector", "load_calibration_tokens", "KNOWN_DATASETS"],
    ".convert": ["convert_model", "should_quantize_tensor", "save_random_checkpoint", "random_hf_state"],
    ".pipeline": ["quantize_checkpoint", "collect_hessians"],
    ".surface": ["BartowskiCalibration", "BartowskiCalibrationV3", "CalibrationBatch", "CalibrationDataset", "CalibrationHooks", "CalibrationStreamer",
                 "EXL3QuantResult", "EXL3Quantizer", "EXL3QuantizerPipeline", "GQACalibrationHooks", "LayerInfo", "LayerStreamer",
                 "LayerStreamerBase", "LayerWeights", "QuantizationResult", "StreamingHessianCollector", "StreamingQuantResult",
                 "StreamingQuantizer", "TrellisCodebook", "TrellisTile", "_HAS_SAFETENSORS", "_HAS_STREAMING", "_HAS_TRANSFORMERS",
                 "analyze_layer_sensitivity", "apply_tensor_core_perm", "apply_tensor_core_perm_i", "blockwise_hadamard",
                 "collect_all_hessians_streaming", "collect_layer_hessian", "compute_model_sensitivity_profile", "compute_quantization_error",
                 "compute_tile_scales", "copy_non_linear_tensors", "ldl_solve", "ldlq_quantize_layer", "ldlq_quantize_layer_core",
                 "load_sensitivity_profile", "preprocess_hessian_exl3", "quantize_model_exl3", "quantize_model_streaming",
                 "quantize_tiles_parallel", "recommend_quantization", "rotate_weights_exl3", "save_exl3_layer", "save_sensitivity_profile",
                 "sensitivity_to_config", "tensor_core_perm", "tensor_core_perm_i", "unrotate_weights_exl3", "quantize_tile_viterbi",
                 "write_exl3_config", "HessianManager"],
}
# adaptive-precision planning objects live with the facade's mixed-precision classes
_COMPAT = ("AdaptiveQuantizer", "AdaptiveQuantResult", "LayerBudget", "ModelBudgetAllocation", "LayerSensitivity", "compute_moe_expert_sensitivity")
_WHERE = {name: mod for mod, names in _MODULES.items() for name in names}


def __getattr__(name: str):
    if name == "pack_indices":
        from ..formats.trellis import pack_codes
        return pack_codes
    if name in _COMPAT:
        from .. import compat_api
        return getattr(compat_api, name)
    mod = _WHERE.get(name)
    if mod is None:
        raise AttributeError(name)
    return getattr(importlib.import_module(mod, __package__), name)


__all__ = sorted(list(_WHERE) + ["pack_indices"] + list(_COMPAT))
