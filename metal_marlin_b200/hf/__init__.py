"""Hugging Face integration: swap ``nn.Linear`` modules of an HF model for quantized layers of this engine, detect MoE
blocks, and load a pre-quantized MMFP4 checkpoint into an HF architecture.

Parity: reference ``metal_marlin/layer_replacement.py`` (``find_linear_layers``, ``replace_linear_layers``,
``find_moe_layers``, ``MetalQuantizedMoE``), ``metal_marlin/model_utils.py:502`` (``load_prequantized_mmfp4_model``:
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


def find_moe_layers(model: nn.Module) -> List[Tuple[str, nn.Module]]:
    """Modules that look like sparse MoE blocks: they own a router (``gate`` / ``router``) and an ``experts`` container."""
    out = []
    for n, m in model.named_modules():
        kids = dict(m.named_children())
        if "experts" in kids and ("gate" in kids or "router" in kids):
            out.append((n, m))
    return out


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


__all__ = ["QuantizedLinearModule", "find_linear_layers", "replace_linear_layers", "find_moe_layers", "load_prequantized_mmfp4_model",
           "DEFAULT_SKIP"]
