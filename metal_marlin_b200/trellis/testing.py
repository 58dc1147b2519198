"""Small random trellis models for tests and demos: linears, dense and MoE MLPs with per-expert bit widths, a decoder layer
and a mini model, all built from seeded random float weights through the real quantizer (nothing here is a stub: the objects
run on the same kernels as loaded checkpoints).

Parity: reference ``trellis/testing.py`` (``create_mock_trellis_linear`` :46, ``create_mock_dense_mlp`` :113, ``create_mock_moe_mlp`` :134,
``create_mini_config`` :179, ``create_mini_model`` :227).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch


def _gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def create_mock_trellis_linear(in_features: int = 128, out_features: int = 64, bits: int = 4, group_size: int = 64, seed: int = 0, device="cpu",
                               std: float = 0.05):
    from ..layers import TrellisLinear
    w = torch.randn(out_features, in_features, generator=_gen(seed)) * std
    return TrellisLinear.from_float(w, bits=bits, group_size=group_size, device=device)


def create_mock_dense_mlp(hidden_size: int = 128, intermediate_size: int = 256, bits: int = 4, group_size: int = 64, seed: int = 0, device="cpu"):
    from .layers import TrellisDenseMLP
    g = _gen(seed)
    mk = lambda o, i: torch.randn(o, i, generator=g) * 0.05      # noqa: E731
    return TrellisDenseMLP.from_float(mk(intermediate_size, hidden_size), mk(intermediate_size, hidden_size), mk(hidden_size, intermediate_size),
                                      bits=bits, group_size=group_size, device=device)


def create_mock_moe_mlp(hidden_size: int = 128, intermediate_size: int = 128, num_experts: int = 4, top_k: int = 2, bits: Sequence[int] = (4,),
                        num_shared_experts: int = 0, group_size: int = 64, seed: int = 0, device="cpu"):
    """``bits``: one width for all experts or one per expert (cycled)."""
    from .layers import MoEConfig, TrellisMoEMLP
    bits = list(bits)
    experts = [create_mock_dense_mlp(hidden_size, intermediate_size, bits[e % len(bits)], group_size, seed * 1000 + e, device) for e in range(num_experts)]
    shared = [create_mock_dense_mlp(hidden_size, intermediate_size, 4, group_size, seed * 1000 + 500 + s, device) for s in range(num_shared_experts)]
    router = torch.randn(num_experts, hidden_size, generator=_gen(seed + 7)).to(device)
    cfg = MoEConfig(num_experts, top_k, hidden_size, intermediate_size, num_shared_experts)
    return TrellisMoEMLP(router, experts, cfg, shared)


def create_mini_config(num_layers: int = 2, hidden_size: int = 128, moe: bool = True, **overrides):
    """A tiny decoder configuration (MLA attention + MoE when ``moe``, a small Llama otherwise)."""
    import dataclasses
    from ..models.config import get_preset
    cfg = get_preset("tiny-mla-moe" if moe else "tiny-llama")
    return dataclasses.replace(cfg, num_hidden_layers=num_layers, **overrides) if (overrides or num_layers != cfg.num_hidden_layers) else cfg


def create_mini_model(config=None, seed: int = 0, device="cpu"):
    """A random-init trellis causal LM over ``config`` (default: :func:`create_mini_config`)."""
    from . import TrellisForCausalLM
    return TrellisForCausalLM.from_config(config or create_mini_config(), device, seed)
