"""INT8 MoE router: the gate matrix ``[num_experts, hidden]`` stored as int8 with one scale per expert row, logits from the
group-quantized kernels (weight-streaming GEMV for decode batches, tcgen05 GEMM with in-loop code expansion above), expert
choice by the one-warp-per-token selection kernel.  A router is read once per token and layer; at int8 it takes a quarter of
its fp32 bytes and half of its bf16 bytes.

Parity: reference ``metal_marlin/trellis/router_int8.py`` (``RouterQuantConfig`` ``:34``, ``Int8RouterLinear`` ``:47`` with
``from_float`` / ``from_weight``, ``Int8Router`` ``:226``, ``quantize_router_weights`` ``:354``,
``measure_quantization_error`` ``:385``).  The reference de-quantizes into a cached float matrix before ``F.linear``; here the
int8 codes are what the kernels read.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from .. import ops
from ..layers.linear import QuantizedLinear
from ..quant.rtn import QuantizedTensor


@dataclass
class RouterQuantConfig:
    per_channel: bool = True          # one scale per expert row (False: one scale for the whole matrix)
    symmetric: bool = True            # the only scheme the kernels' int8 codes use (zero point 128)


def quantize_router_weights(weight: torch.Tensor, config: Optional[RouterQuantConfig] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``weight [E, H]`` -> ``(int8 [E, H], scales fp32 [E])`` with ``scale = max|row| / 127`` (per tensor: one shared value)."""
    config = config or RouterQuantConfig()
    w = weight.detach().to(torch.float32)
    amax = w.abs().amax(dim=1) if config.per_channel else w.abs().max().expand(w.shape[0])
    scales = (amax / 127.0).clamp_min(1e-8)
    q = torch.round(w / scales.unsqueeze(1)).clamp_(-127, 127).to(torch.int8)
    return q, scales.contiguous()


def measure_quantization_error(weight: torch.Tensor, config: Optional[RouterQuantConfig] = None, x: Optional[torch.Tensor] = None,
                               topk: int = 4) -> Dict[str, float]:
    """Weight-space error of the int8 router and, given activations ``x [T, H]``, how often its top-k choice differs."""
    q, s = quantize_router_weights(weight, config)
    w = weight.detach().to(torch.float32)
    wq = q.to(torch.float32) * s.unsqueeze(1)
    out = {"max_abs_error": float((w - wq).abs().max()), "mean_abs_error": float((w - wq).abs().mean()),
           "relative_error": float((w - wq).norm() / w.norm().clamp_min(1e-20))}
    if x is not None:
        a = (x.to(torch.float32) @ w.t()).topk(topk, -1).indices.sort(-1).values
        b = (x.to(torch.float32) @ wq.t()).topk(topk, -1).indices.sort(-1).values
        out["topk_agreement"] = float((a == b).all(-1).float().mean())
    return out


class Int8RouterLinear(QuantizedLinear):
    """``logits = x W^T`` from int8 codes with per-row scales (a ``QuantizedLinear`` whose group is the whole row)."""

    @classmethod
    def from_weight(cls, weight: torch.Tensor, device=None, config: Optional[RouterQuantConfig] = None) -> "Int8RouterLinear":
        q, s = quantize_router_weights(weight, config)
        codes = (q.to(torch.int16) + 128).to(torch.uint8)
        E, H = weight.shape
        # the kernels hold scales in fp16: a power-of-two factor lifts small router scales out of the subnormal range; its
        # inverse goes into the code table and the zero point (w = (table[code] - zero) * scale), so the product is unchanged
        k = int(torch.floor(torch.log2(0.5 / s.max())).item())
        qt = QuantizedTensor(codes, (s * 2.0 ** k).to(torch.float16).view(E, 1), torch.full((E, 1), 128.0, dtype=torch.float16),
                             "int8", H, 8)
        self = cls(qt, None, device if device is not None else weight.device)
        self.lut = self.lut * 2.0 ** -k
        self.zeros = (self.zeros.to(torch.float32) * 2.0 ** -k).to(torch.float16)
        return self

    @classmethod
    def from_float(cls, linear, device=None, config: Optional[RouterQuantConfig] = None) -> "Int8RouterLinear":
        """From an ``nn.Linear``-like module (its ``weight``; routers carry no bias)."""
        return cls.from_weight(linear.weight.data, device, config)


class Int8Router:
    """Gate + expert choice: ``ids, weights = router(x)`` for ``x [T, H]`` with the scoring modes of ``ops.moe_router``
    (softmax or sigmoid + correction bias, group-limited top-k, renormalisation, routed scale)."""

    def __init__(self, gate: Int8RouterLinear, topk: int = 4, scoring: int = 0, renorm: bool = True, routed_scale: float = 1.0,
                 n_group: int = 1, topk_group: int = 1, bias: Optional[torch.Tensor] = None):
        self.gate, self.topk, self.scoring, self.renorm = gate, topk, scoring, renorm
        self.routed_scale, self.n_group, self.topk_group, self.bias = routed_scale, n_group, topk_group, bias

    @property
    def num_experts(self) -> int:
        return self.gate.out_features

    @property
    def hidden_dim(self) -> int:
        return self.gate.in_features

    @classmethod
    def from_weight(cls, weight: torch.Tensor, device=None, **kw) -> "Int8Router":
        return cls(Int8RouterLinear.from_weight(weight, device), **kw)

    @classmethod
    def from_linear(cls, linear, device=None, **kw) -> "Int8Router":
        return cls(Int8RouterLinear.from_float(linear, device), **kw)

    def logits(self, x: torch.Tensor) -> torch.Tensor:
        return self.gate(x.reshape(-1, x.shape[-1])).to(torch.float32)

    def __call__(self, x: torch.Tensor, counts: Optional[torch.Tensor] = None):
        return ops.moe_select(self.logits(x), bias=self.bias, topk=self.topk, scoring=self.scoring, renorm=self.renorm,
                              routed_scale=self.routed_scale, n_group=self.n_group, topk_group=self.topk_group, counts=counts)
