from .deltanet import gated_delta_rule_chunked, gated_delta_rule_recurrent, gated_delta_step, l2norm
from .hybrid import LayerSpec, jamba_layout, kv_layers, layout_from_config, qwen35_layout, zamba_layout
from .mamba import MambaBlock, MambaConfig, mamba2_scan, selective_scan, selective_scan_step
from .rwkv import wkv5, wkv6

__all__ = ["gated_delta_rule_chunked", "gated_delta_rule_recurrent", "gated_delta_step", "l2norm", "LayerSpec", "jamba_layout", "kv_layers",
           "layout_from_config", "qwen35_layout", "zamba_layout", "MambaBlock", "MambaConfig", "mamba2_scan", "selective_scan",
           "selective_scan_step", "wkv5", "wkv6"]
