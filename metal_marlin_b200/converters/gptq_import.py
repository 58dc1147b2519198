"""Import of AutoGPTQ-style INT4 checkpoints (``qweight`` / ``qzeros`` / ``scales`` / ``g_idx``).

Parity: reference ``metal_marlin/converters`` GPTQ importer.  Layout: ``qweight int32 [in / 8, out]`` (eight 4-bit
codes per word along the input axis, LSB first), ``qzeros int32 [in / gs, out / 8]`` (stored minus one),
``scales fp16 [in / gs, out]``, optional ``g_idx int32 [in]`` (group of every input channel, act-order).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch


def dequantize_gptq_int4(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, g_idx: Optional[torch.Tensor] = None,
                         zero_offset: int = 1) -> torch.Tensor:
    """Returns the float weight ``[out, in]``."""
    sh = torch.arange(0, 32, 4, device=qweight.device)
    w = ((qweight.to(torch.int64).unsqueeze(1) >> sh.view(1, 8, 1)) & 0xF).reshape(-1, qweight.shape[1])       # [in, out]
    z = ((qzeros.to(torch.int64).unsqueeze(2) >> sh.view(1, 1, 8)) & 0xF).reshape(qzeros.shape[0], -1) + zero_offset      # [ng, out]
    in_f = w.shape[0]
    if g_idx is None:
        gs = in_f // scales.shape[0]
        g_idx = torch.arange(in_f, device=w.device) // gs
    g = g_idx.long()
    return ((w - z[g]).to(torch.float32) * scales.to(torch.float32)[g]).t().contiguous()


def import_gptq_state(state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Replace every ``<p>.qweight/.qzeros/.scales(/.g_idx)`` quadruple by a float ``<p>.weight``."""
    out: Dict[str, torch.Tensor] = {}
    done = set()
    for k in state:
        if k.endswith(".qweight"):
            p = k[: -len(".qweight")]
            out[p + ".weight"] = dequantize_gptq_int4(state[k], state[p + ".qzeros"], state[p + ".scales"], state.get(p + ".g_idx")).to(torch.bfloat16)
            done.update({k, p + ".qzeros", p + ".scales", p + ".g_idx"})
    for k, v in state.items():
        if k not in done:
            out[k] = v
    return out
