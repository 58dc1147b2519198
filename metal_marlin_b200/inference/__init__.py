"""Inference surface: pipelines, pipelined scheduling, prefill / decode helpers, early exit, long-context helpers and the
tokenizer loader, plus the reference's ``metal_marlin.inference`` names (``MarlinModel``, ``ModelInfo``, ``PrefillModel``,
``TransformersMarlinPipeline``, ``chat``, ``get_device``, ``load_quantized_model``, ``load_safetensors_torch``,
``dequantize_fp4_torch``, ``fused_qkv_projection``, ``batched_kv_projection`` / ``BatchedKVResult``, ``LayerWeights``).
Everything is resolved on first use, so importing the package does not import the model stack."""
from __future__ import annotations

import importlib
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Protocol, Sequence, Tuple

_LAZY = {
    "_fused_sampling": (".generate_loop", "_fused_sampling"), "_optimized_generate": (".generate_loop", "_optimized_generate"),
    "GenerationConfig": ("..trellis", "GenerationConfig"), "MetalMarlinModel": ("..models.mmfp4_causal_lm", "MMFP4ForCausalLM"),
    "ModelConfig": ("..models.config", "ModelConfig"),
    "MMFP4Pipeline": (".pipeline", "MMFP4Pipeline"), "MarlinPipeline": (".pipeline", "MarlinPipeline"),
    "TransformersMarlinPipeline": (".pipeline", "MarlinPipeline"), "StreamingOutput": (".pipeline", "StreamingOutput"),
    "PipelineScheduler": (".pipelined", "PipelineScheduler"), "AsyncPipelineScheduler": (".pipelined", "AsyncPipelineScheduler"),
    "InferenceRequest": (".pipelined", "InferenceRequest"), "RequestState": (".pipelined", "RequestState"),
    "generate_pipelined": (".pipelined", "generate_pipelined"),
    "PrefillConfig": (".prefill", "PrefillConfig"), "PrefillStats": (".prefill", "PrefillStats"), "chunked_prefill": (".prefill", "chunked_prefill"),
    "parallel_kv_write": (".prefill", "parallel_kv_write"), "flash_prefill_attention": (".prefill", "flash_prefill_attention"),
    "SpeculativePrefillConfig": (".prefill", "SpeculativePrefillConfig"), "speculative_prefill": (".prefill", "speculative_prefill"),
    "DecodeConfig": (".decode", "DecodeConfig"), "DecodePerfStats": (".decode", "DecodePerfStats"), "DecodeState": (".decode", "DecodeState"),
    "persistent_decode_step": (".decode", "persistent_decode_step"), "select_decode_kernel": (".decode", "select_decode_kernel"),
    "quantized_kv_attention": (".decode", "quantized_kv_attention"), "quantize_kv_cache": (".decode", "quantize_kv_cache"),
    "EarlyExitModel": (".early_exit", "EarlyExitModel"), "LongContextConfig": (".long_context", "LongContextConfig"),
    "LongContextModel": (".long_context", "LongContextModel"), "load_tokenizer": (".tokenizer", "load_tokenizer"),
    "MarlinModel": ("..models.mmfp4_causal_lm", "MMFP4ForCausalLM"), "LayerWeights": ("..models.transformer", "LayerWeights"),
    "generate": ("..compat_api", "generate"), "generate_stream": ("..compat_api", "generate_stream"), "generate_batch": ("..compat_api", "generate_batch"),
}


def __getattr__(name: str):
    if name in _LAZY:
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod, __package__), attr)
    raise AttributeError(name)


class PrefillModel(Protocol):
    """What the prompt-pass helpers need from a model."""

    def new_cache(self, num_blocks: int, block_size: int = 16, kv_dtype: str = "bf16"): ...

    def forward_logits(self, token_ids: Sequence[int]): ...


@dataclass
class ModelInfo:
    model_type: str
    num_layers: int
    hidden_size: int
    vocab_size: int
    num_attention_heads: int
    num_experts: int
    attention: str
    quant_format: str
    group_size: int
    weight_bytes: int
    device: str
    max_model_len: int

    @classmethod
    def of(cls, pipeline) -> "ModelInfo":
        from .pipeline import MarlinPipeline
        return cls(**(pipeline.info() if hasattr(pipeline, "info") else MarlinPipeline.info(pipeline)))


def get_device(prefer: Optional[str] = None) -> str:
    """``cuda`` (the current device) when a GPU is present, else ``cpu``; an explicit ``prefer`` wins."""
    import torch
    if prefer:
        return prefer
    return f"cuda:{torch.cuda.current_device()}" if torch.cuda.is_available() else "cpu"


def load_safetensors_torch(path: str, device: str = "cpu") -> Dict[str, Any]:
    """All tensors of a safetensors file or of a (sharded) checkpoint directory."""
    import os
    from ..utils.checkpoint import load_checkpoint, load_sharded_checkpoint
    return load_sharded_checkpoint(path, device) if os.path.isdir(path) else load_checkpoint(path, device)


def load_quantized_model(path: str, device: Optional[str] = None):
    """A quantized checkpoint (MMFP4 / marlin FP4 / trellis) as a causal LM of this engine."""
    from ..formats.trellis import detect_trellis_format
    if detect_trellis_format(path) is not None:
        from ..trellis.lm import TrellisForCausalLM
        return TrellisForCausalLM.from_pretrained(path, device=get_device(device))
    from ..models.mmfp4_causal_lm import MMFP4ForCausalLM
    return MMFP4ForCausalLM.from_pretrained(path, get_device(device))


def chat(pipeline, messages: Sequence[Dict[str, str]], **kw) -> str:
    """One chat turn through a pipeline (its chat template, then generation)."""
    return pipeline.chat(messages, **kw)


def dequantize_fp4_torch(packed, scales, K: Optional[int] = None, N: Optional[int] = None, group_size: int = 128):
    """Marlin FP4 ``packed [K / 8, N]`` + ``scales [K / group_size, N]`` -> float ``[K, N]`` (cut to ``K`` x ``N`` when given)."""
    from ..compat_api import unpack_fp4_weights
    import torch
    kp = packed.shape[0] * 8
    meta = {"orig_K": K or kp, "orig_N": N or packed.shape[1], "padded_K": kp, "group_size": kp // scales.shape[0]}
    return unpack_fp4_weights(packed, scales, meta, weights_dtype=torch.float32, output_backend="torch")


def fused_qkv_projection(x, q, k, v):
    """``(packed, scales)`` row-packed MMFP4 pairs for the three projections -> ``(q, k, v)`` outputs from one launch."""
    from ..compat_api import mmfp4_fused_qkv
    return mmfp4_fused_qkv(x, q, k, v)


@dataclass
class BatchedKVResult:
    keys: Any                # [B, T, Hkv, D]
    values: Any              # [B, T, Hkv, D]
    num_tokens: int


def batched_kv_projection(hidden, k_weight, v_weight, num_kv_heads: int, head_dim: int) -> BatchedKVResult:
    """Keys and values of a whole chunk in one projection: ``hidden [B, T, d]`` against the stacked ``[k | v]`` weight (float
    ``[Hkv * D, d]`` matrices or quantized linear layers)."""
    import torch
    B, T, d = hidden.shape
    if callable(k_weight):
        k, v = k_weight(hidden), v_weight(hidden)
    else:
        kv = hidden.reshape(B * T, d).to(k_weight.dtype) @ torch.cat([k_weight, v_weight], 0).t()
        k, v = kv[:, : num_kv_heads * head_dim], kv[:, num_kv_heads * head_dim:]
    return BatchedKVResult(k.reshape(B, T, num_kv_heads, head_dim), v.reshape(B, T, num_kv_heads, -1), B * T)


__all__ = sorted(list(_LAZY) + ["PrefillModel", "ModelInfo", "get_device", "load_safetensors_torch", "load_quantized_model", "chat",
                                "dequantize_fp4_torch", "fused_qkv_projection", "BatchedKVResult", "batched_kv_projection"])
