"""Hugging Face integration: swap ``nn.Linear`` modules of an HF model for quantized layers of this engine, detect MoE
blocks, and load a pre-quantized MMFP4 checkpoint into an HF architecture.

Parity: reference ``metal_marlin/layer_replacement.py`` (``find_linear_layers`` ``:193``, ``replace_linear_layers`` ``:484``,
``find_moe_layers`` ``:206``, ``MetalQuantizedMoE`` ``:50``, ``quantize_moe_experts`` ``:343``, ``replace_moe_layers`` ``:598``,
``replace_moe_layers_streaming`` ``:1469``: one layer at a time with a completion callback), ``metal_marlin/model_utils.py:502`` (``load_prequantized_mmfp4_model``:
model built on the ``meta`` device, quantized tensors attached, norms / router / ``e_score_correction_bias`` copied) and
``metal_marlin/inference_metal.py`` (``MetalQuantizedLinear``).
"""
from __future__ import annotations

import re
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn

from ..layers.linear import MMFP4Linear, QuantizedLinear
from ..ops.weights import FP4Weight

DEFAULT_SKIP = (r"lm_head", r"embed", r"\.gate$", r"router", r"norm")


class QuantizedLinearModule(nn.Module):
    """``nn.Module`` shell around a quantized linear so it can sit inside an HF model (``state_dict`` carries nothing:
    the packed weights are plain tensors owned by the inner layer)."""

    def __init__(self, inner, in_features: int, out_features: int):
        super().__init__()
        self.inner, self.in_features, self.out_features = inner, in_features, out_features

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.inner(x).to(x.dtype)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, kind={type(self.inner).__name__}"


def find_linear_layers(model: nn.Module, skip: Iterable[str] = DEFAULT_SKIP) -> List[Tuple[str, nn.Linear]]:
    pats = [re.compile(p) for p in skip]
    return [(n, m) for n, m in model.named_modules() if isinstance(m, nn.Linear) and not any(p.search(n) for p in pats)]


def _set_module(model: nn.Module, name: str, new: nn.Module) -> None:
    parent = model
    parts = name.split(".")
    for p in parts[:-1]:
        parent = getattr(parent, p)
    setattr(parent, parts[-1], new)


def replace_linear_layers(model: nn.Module, fmt: str = "fp4", group_size: int = 128, skip: Iterable[str] = DEFAULT_SKIP,
                          device=None, min_features: int = 64) -> Dict[str, int]:
    """Quantize every eligible ``nn.Linear`` in place.  Returns counts and the bytes before / after."""
    stats = {"replaced": 0, "skipped": 0, "bytes_before": 0, "bytes_after": 0}
    for name, lin in find_linear_layers(model, skip):
        w = lin.weight.data
        if min(w.shape) < min_features or w.shape[1] % 64:
            stats["skipped"] += 1
            continue
        dev = device or w.device
        bias = None if lin.bias is None else lin.bias.data
        inner = MMFP4Linear.from_float(w.float(), group_size, bias=None if bias is None else bias.to(dev, torch.bfloat16), device=dev) if fmt == "fp4" \
            else QuantizedLinear.from_float(w.float(), fmt, group_size, bias=bias, device=dev)
        stats["bytes_before"] += w.numel() * w.element_size()
        stats["bytes_after"] += inner.weight.nbytes() if fmt == "fp4" else inner.codes.numel() + inner.scales.numel() * 2
        _set_module(model, name, QuantizedLinearModule(inner, lin.in_features, lin.out_features))
        stats["replaced"] += 1
    return stats


class QuantizedMoEExperts(nn.Module):
    """Drop-in for an HF fused experts module (``forward(hidden_states, top_k_index, top_k_weights)``): routed experts held
    as FP4 expert banks (gate rows, then up rows; down), evaluated by this engine's MoE path (per-token weight streaming for a
    few tokens, device-side counting sort + grouped tensor-core GEMMs for many)."""

    def __init__(self, gate_up, down, dtype=torch.bfloat16):
        super().__init__()
        self.gate_up, self.down = gate_up, down
        self.num_experts = gate_up.num_experts
        self.hidden_dim, self.intermediate_dim = gate_up.in_features, down.in_features
        self.out_dtype = dtype

    def forward(self, hidden_states: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor) -> torch.Tensor:
        from .. import ops
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1]).to(torch.bfloat16).contiguous()
        y = ops.moe_forward(x, self.gate_up, self.down, top_k_index.reshape(x.shape[0], -1).to(torch.int32).contiguous(),
                            top_k_weights.reshape(x.shape[0], -1).to(torch.float32).contiguous())
        return y.to(hidden_states.dtype).reshape(shape)

    def extra_repr(self) -> str:
        return f"experts={self.num_experts}, hidden={self.hidden_dim}, intermediate={self.intermediate_dim}, group={self.gate_up.group_size}"


class QuantizedMoEBlock(nn.Module):
    """Drop-in for an HF sparse-MoE block that keeps its experts in a ``ModuleList`` (each with ``gate_proj`` / ``up_proj`` /
    ``down_proj``): the block's own router module stays, the experts become FP4 banks.  Routing follows the block's
    configuration: soft-max over the router logits, top-k, optional renormalisation."""

    def __init__(self, gate: nn.Module, experts: QuantizedMoEExperts, top_k: int, norm_topk_prob: bool, shared: Optional[nn.Module] = None,
                 shared_gate: Optional[nn.Module] = None, returns_router_logits: bool = False):
        super().__init__()
        self.gate, self.experts, self.top_k, self.norm_topk_prob = gate, experts, int(top_k), bool(norm_topk_prob)
        self.shared_expert, self.shared_expert_gate = shared, shared_gate
        self.returns_router_logits = returns_router_logits

    def forward(self, hidden_states: torch.Tensor):
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1])
        logits = self.gate(x)
        if isinstance(logits, tuple):             # routers that already return (logits, weights, indices)
            logits, w, idx = logits
        else:
            probs = torch.softmax(logits.float(), -1)
            w, idx = torch.topk(probs, self.top_k, -1)
            if self.norm_topk_prob:
                w = w / w.sum(-1, keepdim=True)
        y = self.experts(x, idx, w)
        if self.shared_expert is not None:
            sh = self.shared_expert(x)
            if self.shared_expert_gate is not None:
                sh = torch.sigmoid(self.shared_expert_gate(x)) * sh
            y = y + sh
        y = y.reshape(shape)
        return (y, logits) if self.returns_router_logits else y


def _expert_stacks(experts: nn.Module):
    """``(gate_up [E, 2I, H], down [E, H, I])`` float views of an experts container, or ``None`` when its layout is unknown."""
    gu, dn = getattr(experts, "gate_up_proj", None), getattr(experts, "down_proj", None)
    if isinstance(gu, (torch.Tensor, nn.Parameter)) and isinstance(dn, (torch.Tensor, nn.Parameter)) and gu.dim() == 3 and dn.dim() == 3:
        gu, dn = gu.data, dn.data
        E = gu.shape[0]
        if dn.shape[0] != E:
            return None
        # [E, 2I, H] + [E, H, I] (output-major) or [E, H, 2I] + [E, I, H] (input-major): the down matrix tells which
        if gu.shape[1] == 2 * dn.shape[2] and gu.shape[2] == dn.shape[1]:
            return gu, dn
        if gu.shape[2] == 2 * dn.shape[1] and gu.shape[1] == dn.shape[2]:
            return gu.transpose(1, 2), dn.transpose(1, 2)
        return None
    if isinstance(experts, (nn.ModuleList, list, tuple)) and len(experts) and all(hasattr(e, "gate_proj") and hasattr(e, "up_proj")
                                                                                    and hasattr(e, "down_proj") for e in experts):
        gu = torch.stack([torch.cat([e.gate_proj.weight.data, e.up_proj.weight.data], 0) for e in experts])
        dn = torch.stack([e.down_proj.weight.data for e in experts])
        return gu, dn
    return None


def find_moe_layers(model: nn.Module) -> List[Tuple[str, nn.Module]]:
    """Modules that look like sparse MoE blocks: they own a router (``gate`` / ``router``) and an ``experts`` container."""
    out = []
    for n, m in model.named_modules():
        kids = dict(m.named_children())
        if "experts" in kids and ("gate" in kids or "router" in kids):
            out.append((n, m))
    return out


def quantize_moe_experts(experts: nn.Module, group_size: int = 128, device=None) -> Optional[QuantizedMoEExperts]:
    """FP4 banks of one experts container (``None`` if its weight layout is not recognised or not tile aligned)."""
    from ..ops.weights import FP4ExpertBank
    st = _expert_stacks(experts)
    if st is None:
        return None
    gu, dn = st
    H, I = gu.shape[2], dn.shape[2]
    if H % 64 or I % 64 or gu.shape[1] % 32:
        return None
    dev = device or gu.device
    gs_in, gs_mid = (group_size if H % group_size == 0 else 64), (group_size if I % group_size == 0 else 64)
    bank_gu = FP4ExpertBank.from_float(gu.to(dev, torch.float32), gs_in)
    bank_dn = FP4ExpertBank.from_float(dn.to(dev, torch.float32), gs_mid)
    return QuantizedMoEExperts(bank_gu, bank_dn)


def replace_moe_layers_streaming(model: nn.Module, group_size: int = 128, skip: Iterable[str] = (), device=None,
                                 on_layer_complete=None) -> Dict[str, int]:
    """Quantize the MoE blocks one at a time and swap each in as soon as it is done (the float experts of a block are released
    before the next block is touched, so peak memory is one block of float experts plus the quantized model).
    ``on_layer_complete(name, index, total)`` is called after every block."""
    pats = [re.compile(p) for p in skip]
    layers = [(n, m) for n, m in find_moe_layers(model) if not any(p.search(n) for p in pats)]
    stats = {"replaced": 0, "skipped": 0, "experts": 0, "bytes_before": 0, "bytes_after": 0}
    for li, (name, block) in enumerate(layers):
        experts = block.experts
        st = _expert_stacks(experts)
        q = quantize_moe_experts(experts, group_size, device)
        if q is None:
            stats["skipped"] += 1
            continue
        stats["bytes_before"] += sum(t.numel() * t.element_size() for t in st)
        stats["bytes_after"] += q.gate_up.nbytes() + q.down.nbytes()
        stats["experts"] += q.num_experts
        if isinstance(experts, nn.ModuleList):
            cfg = getattr(model, "config", None)
            top_k = getattr(block, "top_k", None) or getattr(cfg, "num_experts_per_tok", 2)
            norm = getattr(block, "norm_topk_prob", None)
            norm = getattr(cfg, "norm_topk_prob", True) if norm is None else norm
            router = getattr(block, "gate", None) or getattr(block, "router")
            new = QuantizedMoEBlock(router, q, top_k, norm, getattr(block, "shared_expert", None), getattr(block, "shared_expert_gate", None),
                                    returns_router_logits=bool(getattr(block, "returns_router_logits", False)))
            _set_module(model, name, new)
        else:
            block.experts = q
        del experts, st
        stats["replaced"] += 1
        if on_layer_complete is not None:
            on_layer_complete(name, li, len(layers))
    return stats


def replace_moe_layers(model: nn.Module, group_size: int = 128, skip: Iterable[str] = (), device=None) -> Dict[str, int]:
    """Quantize every MoE block's routed experts in place (fused 3-D expert tensors or a ``ModuleList`` of expert MLPs)."""
    return replace_moe_layers_streaming(model, group_size, skip, device)


def load_prequantized_mmfp4_model(model: nn.Module, checkpoint_dir: str, device="cpu") -> Dict[str, int]:
    """Attach the tensors of an MMFP4 / marlin_fp4 checkpoint to an HF model instance (typically created on the ``meta``
    device): quantized projections become :class:`QuantizedLinearModule`, everything else (norms, embeddings, router
    weights, ``e_score_correction_bias``) is materialised from the checkpoint."""
    from ..formats.mmfp4_loader import MMFP4ModelLoader
    ld = MMFP4ModelLoader(checkpoint_dir)
    stats = {"quantized": 0, "dense": 0, "missing": 0}
    for name, mod in list(model.named_modules()):
        if isinstance(mod, nn.Linear) and ld.is_quantized(name):
            packed, scales, layout = ld.get_quantized_weight(name)
            w = FP4Weight.from_marlin_fp4(packed, scales, device) if layout == "marlin_fp4" else FP4Weight.from_mmfp4(packed, scales, device)
            bias = ld.load_tensor(name + ".bias").to(device, torch.bfloat16) if ld.has_tensor(name + ".bias") else None
            _set_module(model, name, QuantizedLinearModule(MMFP4Linear(w, bias), mod.in_features, mod.out_features))
            stats["quantized"] += 1
    for pname, p in list(model.named_parameters()) + list(model.named_buffers()):
        if ld.has_tensor(pname):
            t = ld.load_tensor(pname).to(device)
            owner = model
            parts = pname.split(".")
            for q in parts[:-1]:
                owner = getattr(owner, q)
            dtype = p.dtype if p.dtype.is_floating_point else t.dtype
            new = t.to(dtype)
            if isinstance(p, nn.Parameter):
                setattr(owner, parts[-1], nn.Parameter(new, requires_grad=False))
            else:
                owner.register_buffer(parts[-1], new)
            stats["dense"] += 1
        elif p.device.type == "meta":
            stats["missing"] += 1
    # derived, non-persistent buffers (rotary inverse frequencies) are not in any checkpoint: rebuild their modules
    for name, mod in list(model.named_modules()):
        inv = getattr(mod, "inv_freq", None)
        if isinstance(inv, torch.Tensor) and inv.device.type == "meta" and hasattr(model, "config"):
            try:
                _set_module(model, name, type(mod)(config=model.config, device=device))
                stats["missing"] -= 1
            except Exception:
                pass
    return stats


__all__ = ["QuantizedLinearModule", "QuantizedMoEExperts", "QuantizedMoEBlock", "find_linear_layers", "replace_linear_layers", "find_moe_layers",
           "quantize_moe_experts", "replace_moe_layers", "replace_moe_layers_streaming", "load_prequantized_mmfp4_model", "DEFAULT_SKIP"]
