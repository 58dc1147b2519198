"""FLOP calculators for transformer blocks and a per-layer counter.  Parity: reference ``metal_marlin/utils/profile_ops.py``
(``calculate_matmul_flops`` ``:70``, ``calculate_attention_flops`` ``:105``, ``calculate_ffn_flops`` ``:153``,
``calculate_layernorm_flops`` ``:209``, ``calculate_embedding_flops`` ``:229``, ``LayerFLOPs`` ``:36``, ``TransformerLayerFLOPs`` ``:250``,
``LayerFLOPsCounter`` ``:305``, ``profile_model_flops`` ``:493``).  The roofline module (``profiling/roofline.py``) turns these
counts into fractions of the measured peaks."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional


def calculate_matmul_flops(M: int, N: int, K: int, *, quantized: bool = False) -> int:
    """``2 M N K``; a quantized weight adds one multiply per weight element per row block for the scale (``M N K / 16`` as a
    nominal de-quantization cost)."""
    f = 2 * M * N * K
    return f + (M * N * K) // 16 if quantized else f


def calculate_attention_flops(batch: int, seq_len: int, num_heads: int, head_dim: int, *, causal: bool = False,
                              kv_len: Optional[int] = None) -> int:
    """Scores + probabilities x values (``4 B H T N D``, halved for a causal square) plus the soft-max (5 per score)."""
    n = kv_len or seq_len
    pairs = batch * num_heads * seq_len * n
    if causal and n == seq_len:
        pairs = pairs // 2 + batch * num_heads * seq_len // 2
    return 4 * pairs * head_dim + 5 * pairs


def calculate_ffn_flops(batch: int, seq_len: int, hidden_dim: int, ffn_dim: int, *, gated: bool = False, quantized: bool = False) -> int:
    t = batch * seq_len
    mats = 3 if gated else 2
    act = t * ffn_dim * (4 if gated else 1)
    return mats * calculate_matmul_flops(t, ffn_dim, hidden_dim, quantized=quantized) + act


def calculate_layernorm_flops(batch: int, seq_len: int, hidden_dim: int) -> int:
    return 5 * batch * seq_len * hidden_dim


def calculate_embedding_flops(batch: int, seq_len: int, vocab_size: int, hidden_dim: int) -> int:
    """A gather: no arithmetic (the LM head is a matmul and counted as such)."""
    return 0


@dataclass
class LayerFLOPs:
    name: str
    total_flops: int = 0
    matmul_flops: int = 0
    attention_flops: int = 0
    other_flops: int = 0

    def __post_init__(self):
        if not self.total_flops:
            self.total_flops = self.matmul_flops + self.attention_flops + self.other_flops


@dataclass
class TransformerLayerFLOPs:
    attention: int = 0
    projections: int = 0
    ffn: int = 0
    norms: int = 0

    @property
    def total(self) -> int:
        return self.attention + self.projections + self.ffn + self.norms

    @classmethod
    def compute(cls, batch: int, seq_len: int, hidden_dim: int, num_heads: int, ffn_dim: int, *, num_kv_heads: Optional[int] = None,
                gated: bool = True, causal: bool = True, kv_len: Optional[int] = None, quantized: bool = False) -> "TransformerLayerFLOPs":
        t, hd = batch * seq_len, hidden_dim // num_heads
        kvh = num_kv_heads or num_heads
        proj = (calculate_matmul_flops(t, hidden_dim + 2 * kvh * hd, hidden_dim, quantized=quantized)
                + calculate_matmul_flops(t, hidden_dim, hidden_dim, quantized=quantized))
        return cls(calculate_attention_flops(batch, seq_len, num_heads, hd, causal=causal, kv_len=kv_len), proj,
                   calculate_ffn_flops(batch, seq_len, hidden_dim, ffn_dim, gated=gated, quantized=quantized),
                   2 * calculate_layernorm_flops(batch, seq_len, hidden_dim))


class LayerFLOPsCounter:
    """Accumulates named layers; ``summary()`` gives totals and the share of matmuls."""

    def __init__(self):
        self.layers: List[LayerFLOPs] = []

    def add(self, layer: LayerFLOPs) -> None:
        self.layers.append(layer)

    def add_transformer_layer(self, name: str, f: TransformerLayerFLOPs) -> None:
        self.add(LayerFLOPs(name, f.total, f.projections + f.ffn, f.attention, f.norms))

    @property
    def total_flops(self) -> int:
        return sum(l.total_flops for l in self.layers)

    def summary(self) -> Dict[str, float]:
        tot = max(1, self.total_flops)
        return {"layers": len(self.layers), "total_flops": self.total_flops, "total_tflops": self.total_flops / 1e12,
                "matmul_fraction": sum(l.matmul_flops for l in self.layers) / tot,
                "attention_fraction": sum(l.attention_flops for l in self.layers) / tot}


def profile_model_flops(batch: int, seq_len: int, num_layers: int, hidden_dim: int, num_heads: int, ffn_dim: int, vocab_size: int = 0,
                        *, num_kv_heads: Optional[int] = None, gated: bool = True, causal: bool = True, quantized: bool = False
                        ) -> LayerFLOPsCounter:
    c = LayerFLOPsCounter()
    per = TransformerLayerFLOPs.compute(batch, seq_len, hidden_dim, num_heads, ffn_dim, num_kv_heads=num_kv_heads, gated=gated,
                                        causal=causal, quantized=quantized)
    for i in range(num_layers):
        c.add_transformer_layer(f"layer.{i}", per)
    if vocab_size:
        c.add(LayerFLOPs("lm_head", matmul_flops=calculate_matmul_flops(batch * seq_len, vocab_size, hidden_dim)))
    return c
