from .deltanet import gated_delta_rule_chunked, gated_delta_rule_recurrent, gated_delta_step, l2norm
from .hybrid import LayerSpec, jamba_layout, kv_layers, layout_from_config, qwen35_layout, zamba_layout
from .mamba import MambaBlock, MambaConfig, mamba2_scan, selective_scan, selective_scan_step
from .rwkv import wkv5, wkv6
from .blocks import (AttentionLayerConfig, DifferentialAttention, DifferentialAttentionConfig, DifferentialMarlinAttention,
                     HybridArchitectureConfig, HybridBlock, HybridLayerConfig, HybridLayerType, HybridModel, HybridModelBuilder,
                     LayerProtocol, LayerState, MambaLayerConfig, MambaState, MarlinMambaBlock, RWKVBlock, RWKVChannelMixing,
                     RWKVLayerState, RWKVTimeMixing, SelectiveScanConfig, StateType, build_hybrid_config,
                     parse_diff_transformer_config, rwkv_wkv_batched, rwkv_wkv_single_token)

__all__ = ["gated_delta_rule_chunked", "gated_delta_rule_recurrent", "gated_delta_step", "l2norm", "LayerSpec", "jamba_layout", "kv_layers",
           "layout_from_config", "qwen35_layout", "zamba_layout", "MambaBlock", "MambaConfig", "mamba2_scan", "selective_scan",
           "selective_scan_step", "wkv5", "wkv6", "AttentionLayerConfig", "DifferentialAttention", "DifferentialAttentionConfig",
           "DifferentialMarlinAttention", "HybridArchitectureConfig", "HybridBlock", "HybridLayerConfig", "HybridLayerType", "HybridModel",
           "HybridModelBuilder", "LayerProtocol", "LayerState", "MambaLayerConfig", "MambaState", "MarlinMambaBlock", "RWKVBlock",
           "RWKVChannelMixing", "RWKVLayerState", "RWKVTimeMixing", "SelectiveScanConfig", "StateType", "build_hybrid_config",
           "parse_diff_transformer_config", "rwkv_wkv_batched", "rwkv_wkv_single_token"]


def __getattr__(name: str):
    if name == "create_causal_mask":                 # the differential-attention module of the reference re-exports the mask helper
        from ..compat_api import create_causal_mask
        return create_causal_mask
    raise AttributeError(name)


__all__ += ["create_causal_mask"]
