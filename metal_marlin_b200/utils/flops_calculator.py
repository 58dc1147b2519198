"""Per-module FLOP accounting: FLOPs of a layer by type, of a quantized linear (with its de-quantization work itemised), and a
calculator that walks a ``torch.nn`` model, a tree of this package's layer objects, or an engine model's configuration.

Counting rules: a matrix product is ``2 M N K``; a 4-bit weight adds one multiply per weight element per token-tile of 128
rows for the scale (the kernels de-quantize a weight tile once per 128-row tile of activations, not per row); a bias adds
``M N``.  Attention is ``4 B H T N D`` (halved for a causal square) plus 5 per score for the soft-max.

Parity: reference ``profile/calculator.py`` (``LayerProfileConfig`` :26, ``ModuleFLOPsResult`` :47, ``estimate_marlin_linear_flops`` :81,
``calculate_layer_flops`` :135, ``LayerFLOPsCalculator`` :225, ``profile_model_layers`` :464).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .profile_ops import calculate_attention_flops, calculate_embedding_flops, calculate_ffn_flops, calculate_layernorm_flops

DEQUANT_ROW_TILE = 128


@dataclass
class LayerProfileConfig:
    batch_size: int = 1
    seq_len: int = 2048
    quantized: bool = True
    group_size: int = 128
    causal_attention: bool = True
    gated_ffn: bool = True


@dataclass
class ModuleFLOPsResult:
    name: str
    module_type: str
    flops: int
    params: int = 0
    input_shape: Optional[Tuple[int, ...]] = None
    output_shape: Optional[Tuple[int, ...]] = None
    metadata: Dict[str, Any] = field(default_factory=dict)

    @property
    def tflops(self) -> float:
        return self.flops / 1e12

    @property
    def gflops(self) -> float:
        return self.flops / 1e9


def estimate_marlin_linear_flops(in_features: int, out_features: int, batch_size: int = 1, seq_len: int = 1, quantized: bool = True,
                                 group_size: int = 128, include_bias: bool = True) -> int:
    rows = batch_size * seq_len
    flops = 2 * rows * in_features * out_features
    if quantized:
        tiles = -(-rows // DEQUANT_ROW_TILE)
        flops += tiles * in_features * out_features                 # code -> value times group scale, once per row tile
    if include_bias:
        flops += rows * out_features
    return int(flops)


def calculate_layer_flops(layer_type: str, **kw: Any) -> int:
    """``linear`` (``in_features``, ``out_features``, ``batch_size``, ``seq_len``, ``quantized``, ``group_size``, ``include_bias``), ``attention``
    (``batch_size``, ``seq_len``, ``num_heads``, ``head_dim``, ``causal``, ``kv_len``), ``ffn`` (``batch_size``, ``seq_len``, ``hidden_dim``, ``ffn_dim``,
    ``gated``, ``quantized``), ``layernorm`` / ``rmsnorm`` (``batch_size``, ``seq_len``, ``hidden_dim``), ``embedding``."""
    t = layer_type.lower()
    b, s = kw.pop("batch_size", 1), kw.pop("seq_len", 1)
    if t in ("linear", "marlin_linear", "quantized_linear"):
        return estimate_marlin_linear_flops(kw["in_features"], kw["out_features"], b, s, kw.get("quantized", True), kw.get("group_size", 128),
                                            kw.get("include_bias", False))
    if t == "attention":
        return calculate_attention_flops(b, s, kw["num_heads"], kw["head_dim"], causal=kw.get("causal", False), kv_len=kw.get("kv_len"))
    if t in ("ffn", "mlp"):
        return calculate_ffn_flops(b, s, kw["hidden_dim"], kw["ffn_dim"], gated=kw.get("gated", False), quantized=kw.get("quantized", False))
    if t in ("layernorm", "rmsnorm", "norm"):
        return calculate_layernorm_flops(b, s, kw["hidden_dim"])
    if t == "embedding":
        return calculate_embedding_flops(b, s, kw.get("vocab_size", 0), kw.get("hidden_dim", 0))
    raise ValueError(f"unknown layer type {layer_type!r} (linear, attention, ffn, layernorm, embedding)")


class LayerFLOPsCalculator:
    def __init__(self, batch_size: int = 1, seq_len: int = 2048, quantized: bool = True, group_size: int = 128, causal_attention: bool = True,
                 gated_ffn: bool = True):
        self.config = LayerProfileConfig(batch_size, seq_len, quantized, group_size, causal_attention, gated_ffn)
        self._results: List[ModuleFLOPsResult] = []

    def _rows(self, input_shape) -> Tuple[int, int]:
        if input_shape is not None and len(input_shape) >= 2:
            rows = 1
            for d in input_shape[:-1]:
                rows *= int(d)
            return rows, 1
        return self.config.batch_size, self.config.seq_len

    def _analyze(self, name: str, module: Any, input_shape) -> Optional[ModuleFLOPsResult]:
        import torch.nn as nn
        b, s = self._rows(input_shape)
        c = self.config
        kind = type(module).__name__
        in_f, out_f = getattr(module, "in_features", None), getattr(module, "out_features", None)
        if isinstance(module, nn.Linear):
            flops = estimate_marlin_linear_flops(in_f, out_f, b, s, quantized=False, include_bias=module.bias is not None)
            return ModuleFLOPsResult(name, kind, flops, sum(p.numel() for p in module.parameters()), input_shape, None, {"quantized": False})
        if in_f is not None and out_f is not None:                      # this package's linear layer objects and quantized modules
            gs = int(getattr(module, "group_size", c.group_size) or c.group_size)
            bias = getattr(module, "bias", None) is not None
            flops = estimate_marlin_linear_flops(int(in_f), int(out_f), b, s, quantized=True, group_size=gs, include_bias=bias)
            return ModuleFLOPsResult(name, kind, flops, int(in_f) * int(out_f), input_shape, None, {"quantized": True, "group_size": gs})
        if isinstance(module, (nn.LayerNorm, nn.RMSNorm)):
            h = int(module.normalized_shape[-1])
            return ModuleFLOPsResult(name, kind, calculate_layernorm_flops(b, s, h), sum(p.numel() for p in module.parameters()), input_shape)
        if isinstance(module, nn.Embedding):
            return ModuleFLOPsResult(name, kind, 0, module.weight.numel(), input_shape)
        if isinstance(module, nn.MultiheadAttention):
            hd = module.embed_dim // module.num_heads
            proj = 4 * estimate_marlin_linear_flops(module.embed_dim, module.embed_dim, b, s, quantized=False, include_bias=module.in_proj_bias is not None)
            att = calculate_attention_flops(b, s, module.num_heads, hd, causal=c.causal_attention)
            return ModuleFLOPsResult(name, kind, proj + att, sum(p.numel() for p in module.parameters()), input_shape, None, {"attention_flops": att})
        return None

    def add_module(self, name: str, module: Any, input_shape: Optional[Tuple[int, ...]] = None) -> Optional[ModuleFLOPsResult]:
        try:
            r = self._analyze(name, module, input_shape)
        except Exception:
            return None
        if r is not None:
            self._results.append(r)
        return r

    def add_layer(self, name: str, layer_type: str, params: int = 0, **kw) -> ModuleFLOPsResult:
        kw.setdefault("batch_size", self.config.batch_size)
        kw.setdefault("seq_len", self.config.seq_len)
        meta = dict(kw)
        r = ModuleFLOPsResult(name, layer_type, calculate_layer_flops(layer_type, **kw), params, metadata=meta)
        self._results.append(r)
        return r

    def add_model_config(self, cfg) -> "LayerFLOPsCalculator":
        """The decoder described by a :class:`models.config.ModelConfig`: per layer the attention projections, the score /
        value products and the MLP (for MoE layers the routed experts a token uses, the shared experts and the router), plus
        the LM head."""
        c = self.config
        h, hd = cfg.hidden_size, cfg.head_dim or cfg.hidden_size // cfg.num_attention_heads
        nq, nkv = cfg.num_attention_heads, cfg.num_key_value_heads or cfg.num_attention_heads
        lin = lambda n, i, o: self.add_layer(n, "linear", i * o, in_features=i, out_features=o, quantized=c.quantized, group_size=c.group_size)   # noqa: E731
        for l in range(cfg.num_hidden_layers):
            p = f"layers.{l}"
            if getattr(cfg, "is_mla", False):
                qk = cfg.qk_nope_head_dim + cfg.qk_rope_head_dim
                if cfg.q_lora_rank:
                    lin(f"{p}.attn.q_a", h, cfg.q_lora_rank)
                    lin(f"{p}.attn.q_b", cfg.q_lora_rank, nq * qk)
                else:
                    lin(f"{p}.attn.q", h, nq * qk)
                lin(f"{p}.attn.kv_a", h, cfg.kv_lora_rank + cfg.qk_rope_head_dim)
                lin(f"{p}.attn.kv_b", cfg.kv_lora_rank, nq * (cfg.qk_nope_head_dim + cfg.v_head_dim))
                lin(f"{p}.attn.o", nq * cfg.v_head_dim, h)
                self.add_layer(f"{p}.attn.core", "attention", num_heads=nq, head_dim=(qk + cfg.v_head_dim) // 2, causal=c.causal_attention)
            else:
                lin(f"{p}.attn.qkv", h, (nq + 2 * nkv) * hd)
                lin(f"{p}.attn.o", nq * hd, h)
                self.add_layer(f"{p}.attn.core", "attention", num_heads=nq, head_dim=hd, causal=c.causal_attention)
            moe = bool(getattr(cfg, "num_experts", 0)) and cfg.layer_is_moe(l)
            if moe:
                k, inter = cfg.num_experts_per_tok, cfg.moe_intermediate_size or cfg.intermediate_size
                lin(f"{p}.moe.router", h, cfg.num_experts).metadata["quantized"] = False
                for tag, n in (("routed", k), ("shared", int(getattr(cfg, "n_shared_experts", 0) or 0))):
                    if n:
                        r = self.add_layer(f"{p}.moe.{tag}", "ffn", 3 * h * inter * (cfg.num_experts if tag == "routed" else n), hidden_dim=h,
                                           ffn_dim=inter * n, gated=True, quantized=c.quantized)
                        r.metadata["experts_per_token"] = n
            else:
                self.add_layer(f"{p}.mlp", "ffn", 3 * h * cfg.intermediate_size, hidden_dim=h, ffn_dim=cfg.intermediate_size, gated=c.gated_ffn,
                               quantized=c.quantized)
            self.add_layer(f"{p}.norms", "rmsnorm", 2 * h, hidden_dim=2 * h)
        lin("lm_head", h, cfg.vocab_size)
        return self

    @property
    def total_flops(self) -> int:
        return sum(r.flops for r in self._results)

    @property
    def total_params(self) -> int:
        return sum(r.params for r in self._results)

    @property
    def total_tflops(self) -> float:
        return self.total_flops / 1e12

    def get_results(self) -> List[ModuleFLOPsResult]:
        return list(self._results)

    def get_layer(self, name: str) -> Optional[ModuleFLOPsResult]:
        return next((r for r in self._results if r.name == name), None)

    def summary_text(self, top_n: int = 20) -> str:
        c = self.config
        lines = [f"FLOPs at batch {c.batch_size} x {c.seq_len} tokens: {self.total_tflops:.4f} TFLOP over {len(self._results)} modules, "
                 f"{self.total_params / 1e6:.1f} M parameters"]
        total = max(1, self.total_flops)
        for r in sorted(self._results, key=lambda r: -r.flops)[:top_n]:
            lines.append(f"  {r.name:<40} {r.module_type:<22} {r.gflops:>12.3f} GFLOP  {100.0 * r.flops / total:5.1f} %")
        return "\n".join(lines)

    def print_summary(self, top_n: int = 20) -> None:
        print(self.summary_text(top_n))

    def clear(self) -> None:
        self._results = []


def profile_model_layers(model: Any, batch_size: int = 1, seq_len: int = 2048, quantized: bool = True) -> LayerFLOPsCalculator:
    """``model``: a ``torch.nn.Module`` (its leaf modules), an engine model (anything with a ``config`` that is a ``ModelConfig``), or
    a ``ModelConfig`` itself."""
    from ..models.config import ModelConfig
    calc = LayerFLOPsCalculator(batch_size, seq_len, quantized)
    cfg = model if isinstance(model, ModelConfig) else getattr(model, "config", None)
    if isinstance(cfg, ModelConfig):
        return calc.add_model_config(cfg)
    for name, mod in model.named_modules():
        if not list(mod.children()) or type(mod).__name__ == "MultiheadAttention":
            calc.add_module(name, mod)
    return calc
