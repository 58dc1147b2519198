"""Trellis building blocks under the reference's names: index packing, de-quantization and GEMM dispatch functions, layer
objects (dense MLP, expert, MoE MLP with mixed bit widths per expert, MLA attention, decoder layer), caches and mixed-bit
dispatch statistics.  The whole-model path (``TrellisForCausalLM``) runs on the shared decoder; these objects serve code
that assembles layers by hand.

Parity: reference ``metal_marlin/trellis/packing.py`` (``pack_indices*``, ``unpack_indices*``, ``pack_trellis_indices``,
``unpack_trellis_indices``, ``compute_packed_size``, ``compute_compression_ratio``), ``trellis/dispatch.py`` (``dispatch_trellis_dequant*``,
``dispatch_gemm_trellis_auto``, ``dispatch_gemm_trellis_decode_auto``, ``dispatch_sign_flips``, ``dequantize_trellis_weight``),
``trellis/mixed_bpw_dispatch.py`` (``MixedBPWMoEDispatcher``, ``dispatch_mixed_bpw_moe``, statistics), ``trellis/layer.py`` / ``moe.py`` /
``attention.py`` / ``model.py`` (``TrellisDenseMLP``, ``TrellisExpert``, ``TrellisMoEMLP``, ``TrellisMoELayer``, ``TrellisMLAttention``,
``TrellisMLAConfig``, ``create_mla_projections``, ``TrellisDecoderLayer``, ``TrellisKVCache``, ``CompressedKVCache``, ``CausalLMOutput``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import ops
from ..formats import trellis as trfmt
from ..kv.contiguous import MLAKVCache
from ..layers.blocks import MMFP4MLA
from ..layers.linear import TrellisLinear
from ..ops.generic import GenericExpertBank
from ..ops.generic import moe_forward as _generic_moe

GLM4_TOKENIZER_ID = "zai-org/GLM-4.7-Flash"
TrellisKVCache = MLAKVCache


class CompressedKVCache(MLAKVCache):
    """The latent cache with 8-bit storage by default (a quarter of the bytes of bf16 keys and values of the heads it stands
    for, on top of the latent compression itself)."""

    def __init__(self, num_layers: int, kv_lora_rank: int, rope_dim: int, batch_size: int = 1, max_seq_len: int = 4096, dtype: str = "fp8", **kw):
        super().__init__(num_layers, kv_lora_rank, rope_dim, batch_size, max_seq_len, dtype, **kw)


@dataclass
class CausalLMOutput:
    logits: torch.Tensor
    past_key_values: Any = None
    hidden_states: Optional[torch.Tensor] = None


# ------------------------------------------------------------------------------------------------ packing
def pack_indices(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """``codes uint8 [out, in]`` (values < 2**bits) -> the checkpoint blob (header byte + 16 x 16 tiles, LSB-first bit stream)."""
    return trfmt.pack_codes(codes, bits)


pack_indices_vectorized = pack_indices
pack_trellis_indices = pack_indices


def unpack_indices(indices: torch.Tensor, out_features: int, in_features: int) -> torch.Tensor:
    return trfmt.unpack_codes(indices, out_features, in_features)[0]


unpack_indices_vectorized = unpack_indices
unpack_trellis_indices = unpack_indices


def compute_packed_size(out_features: int, in_features: int, bits: int) -> int:
    """Bytes of the index blob: one header byte plus ``32 * bits`` bytes per 16 x 16 tile."""
    tiles = -(-out_features // 16) * -(-in_features // 16)
    return 1 + tiles * trfmt.tile_bytes(bits)


def compute_compression_ratio(out_features: int, in_features: int, bits: int, group_size: int = 128) -> float:
    """fp16 bytes over trellis bytes (indices + fp32 group scales + the two sign vectors)."""
    dense = 2.0 * out_features * in_features
    packed = compute_packed_size(out_features, in_features, bits) + 4.0 * (-(-in_features // group_size) * out_features + in_features + out_features)
    return dense / packed


# ------------------------------------------------------------------------------------------------ de-quantization and GEMM dispatch
def dequantize_trellis_weight(weight, dtype=torch.float32) -> torch.Tensor:
    """``TrellisWeight`` (checkpoint form) or ``TrellisLinear`` (device form) -> float ``[out, in]``."""
    return weight.dequantize(dtype)


def dispatch_trellis_dequant(codes: torch.Tensor, scales: torch.Tensor, su: torch.Tensor, sv: torch.Tensor, out_features: int,
                             in_features: int, bits: int, group_size: int = 128) -> torch.Tensor:
    """Header-less code stream + scales ``[groups, out]`` + sign vectors -> bf16 ``[out, in]`` (the de-quantization kernel)."""
    return ops.trellis_dequant(codes, scales, su, sv, out_features, in_features, bits, group_size)


dispatch_trellis_dequant_fused = dispatch_trellis_dequant
dispatch_trellis_dequant_packed = dispatch_trellis_dequant


def dispatch_sign_flips(x: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
    """Multiply the last axis by a +-1 vector (the random sign flips in front of / behind a trellis matrix)."""
    return x * signs.to(x.dtype)


def dispatch_gemm_trellis_auto(x: torch.Tensor, layer: TrellisLinear) -> torch.Tensor:
    """``x @ W^T`` by token count: bit-stream GEMV for decode batches, tcgen05 GEMM with in-loop decoding above."""
    return layer(x)


dispatch_gemm_trellis_decode_auto = dispatch_gemm_trellis_auto


# ------------------------------------------------------------------------------------------------ layer objects
class TrellisDenseMLP:
    """SwiGLU MLP over three trellis matrices (any bit width each)."""

    def __init__(self, gate: TrellisLinear, up: TrellisLinear, down: TrellisLinear):
        self.gate, self.up, self.down = gate, up, down
        self.in_features, self.out_features = gate.in_features, down.out_features

    @classmethod
    def from_float(cls, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, bits=4, group_size: int = 128, device=None) -> "TrellisDenseMLP":
        b = (bits, bits, bits) if isinstance(bits, int) else tuple(bits)
        return cls(*(TrellisLinear.from_float(w, bb, group_size, device) for w, bb in zip((gate, up, down), b)))

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.down((F.silu(self.gate(x).float()) * self.up(x).float()).to(torch.bfloat16)).to(x.dtype)


TrellisExpert = TrellisDenseMLP


class _GateUp:
    """gate | up of one expert as one callable ``[M, H] -> [M, 2 I]`` (what the generic expert bank expects)."""
    is_generic = True

    def __init__(self, gate: TrellisLinear, up: TrellisLinear):
        self.gate, self.up = gate, up
        self.in_features, self.out_features = gate.in_features, gate.out_features + up.out_features
        self.parts = [gate, up]

    def __call__(self, x):
        return torch.cat([self.gate(x), self.up(x)], -1)


_stats = {"calls": 0, "tokens": 0, "by_bits": {}}


def get_mixed_bpw_stats() -> Dict[str, Any]:
    return {"calls": _stats["calls"], "tokens": _stats["tokens"], "by_bits": dict(_stats["by_bits"])}


def reset_mixed_bpw_stats() -> None:
    _stats.update(calls=0, tokens=0, by_bits={})


@dataclass
class MoEConfig:
    num_experts: int
    top_k: int
    hidden_size: int
    intermediate_size: int
    num_shared_experts: int = 0
    scoring: str = "softmax"
    renormalize: bool = True
    routed_scale: float = 1.0


class TrellisMoEMLP:
    """Router + trellis experts (bit widths may differ per expert and per matrix) + optional shared experts, on the generic
    MoE path: two device-side launches for decode batches, counting sort + grouped tensor-core GEMMs for prompts."""

    def __init__(self, router_weight: torch.Tensor, experts: Sequence[TrellisDenseMLP], config: MoEConfig,
                 shared: Sequence[TrellisDenseMLP] = (), correction_bias: Optional[torch.Tensor] = None):
        from ..ops.generic import CatWeight
        self.cfg, self.router_weight, self.correction_bias = config, router_weight.to(torch.bfloat16), correction_bias
        allx = list(experts) + list(shared)
        self.bank = GenericExpertBank([CatWeight([e.gate, e.up]) for e in allx], [e.down for e in allx])
        self.experts, self.shared = list(experts), list(shared)

    def route(self, x: torch.Tensor):
        c = self.cfg
        return ops.moe_router(x, self.router_weight, bias=self.correction_bias, topk=c.top_k, scoring={"softmax": 0, "sigmoid": 1}[c.scoring],
                              renorm=c.renormalize, routed_scale=c.routed_scale)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(torch.bfloat16).contiguous()
        ids, w = self.route(x2)
        _stats["calls"] += 1
        _stats["tokens"] += x2.shape[0]
        for e in ids.reshape(-1).tolist():
            b = self.experts[e].gate.bits
            _stats["by_bits"][b] = _stats["by_bits"].get(b, 0) + 1
        y = _generic_moe(x2, self.bank, ids, w, n_shared=len(self.shared), shared_base=len(self.experts))
        return y.view(shape).to(x.dtype)


TrellisMoELayer = TrellisMoEMLP
MixedBPWMoEDispatcher = TrellisMoEMLP


def dispatch_mixed_bpw_moe(x: torch.Tensor, moe: TrellisMoEMLP) -> torch.Tensor:
    return moe(x)


dispatch_mixed_bpw_moe_with_cpp_fallback = dispatch_mixed_bpw_moe


@dataclass
class TrellisMLAConfig:
    hidden_size: int
    num_heads: int
    q_lora_rank: int
    kv_lora_rank: int
    qk_nope_head_dim: int
    qk_rope_head_dim: int
    v_head_dim: int
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    rope_interleave: bool = True


def create_mla_projections(config: TrellisMLAConfig, state: Dict[str, torch.Tensor], bits: int = 4, group_size: int = 128, device=None
                           ) -> Dict[str, object]:
    """Float tensors ``q_a_proj``, ``q_a_layernorm``, ``q_b_proj``, ``kv_a_proj_with_mqa``, ``kv_a_layernorm``, ``kv_b_proj``, ``o_proj`` ->
    the trellis projections and norm vectors of an MLA layer."""
    lin = lambda n: TrellisLinear.from_float(state[n].float(), bits, group_size, device)
    dev = device or state["q_a_proj"].device
    return {"q_a": lin("q_a_proj"), "q_a_norm": state["q_a_layernorm"].to(dev), "q_b": lin("q_b_proj"), "kv_a": lin("kv_a_proj_with_mqa"),
            "kv_a_norm": state["kv_a_layernorm"].to(dev), "kv_b": lin("kv_b_proj"), "o": lin("o_proj")}


class TrellisMLAttention(MMFP4MLA):
    """Multi-head latent attention over trellis projections (requires the low-rank query path, like the reference)."""

    def __init__(self, config: TrellisMLAConfig, projections: Dict[str, object]):
        if "q_a" not in projections or "q_b" not in projections:
            raise ValueError("TrellisMLAttention needs q_a / q_b projections (MLA with a low-rank query path)")
        super().__init__(projections, config.num_heads, config.qk_nope_head_dim, config.qk_rope_head_dim, config.v_head_dim,
                         config.kv_lora_rank, config.rope_theta, config.rms_norm_eps, config.rope_interleave)
        self.config = config


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


class TrellisDecoderLayer:
    """Pre-norm decoder layer: ``x + attn(norm(x))`` then ``x + mlp(norm(x))`` (``mlp``: dense or MoE)."""

    def __init__(self, attention, mlp, input_norm: torch.Tensor, post_attention_norm: torch.Tensor, eps: float = 1e-6):
        self.attention, self.mlp, self.input_norm, self.post_norm, self.eps = attention, mlp, input_norm, post_attention_norm, eps

    def __call__(self, x: torch.Tensor, positions: Optional[torch.Tensor] = None, cache=None, layer: int = 0) -> torch.Tensor:
        x = x + self.attention(_rms(x, self.input_norm, self.eps), positions, cache, layer).to(x.dtype)
        return x + self.mlp(_rms(x, self.post_norm, self.eps)).to(x.dtype)
