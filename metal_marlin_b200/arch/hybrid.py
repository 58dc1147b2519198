"""Hybrid layer layouts: which layer of a stack is attention, Mamba, DeltaNet or MoE.

Parity: reference ``metal_marlin/architectures/hybrid.py`` (Jamba: one attention layer per period of Mamba layers, MoE
every other layer; Zamba: a shared attention block re-applied every N Mamba layers) and the Qwen3.5 / 3.6 pattern
(three Gated DeltaNet layers then one full-attention layer).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional


@dataclass(frozen=True)
class LayerSpec:
    mixer: str            # "attention" | "mamba" | "deltanet" | "shared_attention"
    mlp: str              # "dense" | "moe"


def jamba_layout(n_layers: int, attn_period: int = 8, attn_offset: int = 4, moe_period: int = 2, moe_offset: int = 1) -> List[LayerSpec]:
    return [LayerSpec("attention" if i % attn_period == attn_offset else "mamba", "moe" if i % moe_period == moe_offset else "dense")
            for i in range(n_layers)]


def zamba_layout(n_layers: int, shared_every: int = 6) -> List[LayerSpec]:
    return [LayerSpec("shared_attention" if (i + 1) % shared_every == 0 else "mamba", "dense") for i in range(n_layers)]


def qwen35_layout(n_layers: int, full_attention_interval: int = 4, moe: bool = True) -> List[LayerSpec]:
    return [LayerSpec("attention" if (i + 1) % full_attention_interval == 0 else "deltanet", "moe" if moe else "dense") for i in range(n_layers)]


def layout_from_config(cfg: dict) -> List[LayerSpec]:
    """Build from HF-style config fields: ``layer_types`` (explicit list), or ``full_attention_interval``, or Jamba's
    ``attn_layer_period`` / ``attn_layer_offset`` / ``expert_layer_period`` / ``expert_layer_offset``."""
    n = int(cfg["num_hidden_layers"])
    if cfg.get("layer_types"):
        names = {"linear_attention": "deltanet", "full_attention": "attention", "mamba": "mamba", "attention": "attention"}
        moe = bool(cfg.get("num_experts") or cfg.get("n_routed_experts"))
        return [LayerSpec(names.get(t, t), "moe" if moe else "dense") for t in cfg["layer_types"]]
    if cfg.get("full_attention_interval"):
        return qwen35_layout(n, int(cfg["full_attention_interval"]), bool(cfg.get("num_experts")))
    if cfg.get("attn_layer_period"):
        return jamba_layout(n, int(cfg["attn_layer_period"]), int(cfg.get("attn_layer_offset", 0)), int(cfg.get("expert_layer_period", 2)),
                            int(cfg.get("expert_layer_offset", 1)))
    return [LayerSpec("attention", "moe" if cfg.get("num_experts") else "dense") for _ in range(n)]


def kv_layers(layout: List[LayerSpec]) -> List[int]:
    """Indices of layers that need a KV cache (recurrent layers keep a fixed-size state instead)."""
    return [i for i, l in enumerate(layout) if l.mixer in ("attention", "shared_attention")]
