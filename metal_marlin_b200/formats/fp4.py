"""FP4 (E2M1) group-quantized weight layouts: checkpoint layouts and the device tile layout.

Checkpoint layouts (loaded unchanged):

* ``marlin_fp4``: packed ``uint32 [in/8, out]`` (eight E2M1 nibbles along the input
  axis per word, nibble *i* in bits ``4i..4i+3`` is element ``8j+i``), scales
  ``fp16 [in/gs, out]``.  Parity: reference ``metal_marlin/quantize_fp4.py:131``
  and ``metal_marlin/hf_loader.py:424-606``.
* ``mmfp4`` (``mmfp4_e2m1_marlin``): packed ``uint32 [out, in/8]`` (row packed, same
  nibble order), scales ``fp16 [out, in/gs]`` (or transposed; both are accepted).
  Parity: reference ``metal_marlin/mr_gptq.py:620-649`` and
  ``metal_marlin/layers/mmfp4_linear.py:695-711``.

Device tile layout (what the sm_100a kernels read; built once at load time):

* weights ``int32 [out/16, in/64, 32, 4]``.  Block ``(rt, kc)`` holds rows
  ``16*rt .. 16*rt+15`` and input columns ``64*kc .. 64*kc+63``; the four words of
  lane ``l = 4*g + t`` are the four k16 steps of that block, and the eight nibbles
  of each word are exactly the lane's A-fragment of an ``m16n8k16`` MMA.  Inside each
  16-bit half the four sign bits sit in bits 15..12 (fragment register 0..3) and the
  four 3-bit magnitudes in bits 11..9, 8..6, 5..3, 2..0, so register ``j`` is
  ``((w << j) & 0x80008000) | ((w << 3j) & 0x0E000E00)``: four independent
  extractions from the same word (no serial shift chain), register 0 with a single
  AND.  A warp reads one block with a single coalesced 512-byte load and needs no
  shuffles.
* scales ``fp16 [out/16, in/gs, 8, 2]``: the two scales a lane needs (rows ``g`` and
  ``g+8``) sit in one 32-bit word.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from .._compat import E2M1_VALUES, get_e2m1_torch_table

_MAG_BOUNDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def pick_group_size(in_features: int, group_size: int) -> int:
    """Largest of (group_size, 64, 32, 16, 8) dividing ``in_features``.
    Parity: reference ``metal_marlin/hf_loader.py:515-524``."""
    if in_features % group_size == 0:
        return group_size
    for gs in (64, 32, 16, 8):
        if gs < group_size and in_features % gs == 0:
            return gs
    raise ValueError(f"in_features={in_features} is not divisible by any supported group size")


def quantize_codes(w: torch.Tensor, group_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """Round-to-nearest E2M1 quantization of ``w [out, in]``.

    Returns ``codes uint8 [out, in]`` and ``scales fp16 [out, in/gs]`` with
    ``scale = absmax / 6`` per group (the reference's rule)."""
    assert w.dim() == 2
    out_f, in_f = w.shape
    assert in_f % group_size == 0, (in_f, group_size)
    wf = w.detach().to(torch.float32)
    g = wf.view(out_f, in_f // group_size, group_size)
    absmax = g.abs().amax(dim=-1)
    scales = (absmax / 6.0).to(torch.float16)
    # A zero (or underflowed) scale would divide by zero; the smallest fp16 subnormal keeps the group ~0.
    scales = torch.where(scales > 0, scales, torch.full_like(scales, 6e-8))
    sf = scales.to(torch.float32).unsqueeze(-1)
    x = (g / sf).clamp_(-6.0, 6.0)
    bounds = torch.tensor(_MAG_BOUNDS, dtype=torch.float32, device=w.device)
    mag = torch.bucketize(x.abs(), bounds)            # 0..7
    sign = (x < 0) & (mag > 0)
    codes = (mag + sign.to(mag.dtype) * 8).to(torch.uint8).view(out_f, in_f)
    return codes, scales


def dequantize_codes(codes: torch.Tensor, scales: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """``W[o, i] = E2M1[codes[o, i]] * scales[o, i // gs]`` in ``dtype``."""
    out_f, in_f = codes.shape
    n_groups = scales.shape[1]
    gs = in_f // n_groups
    table = get_e2m1_torch_table(codes.device, torch.float32)
    vals = table[codes.long()].view(out_f, n_groups, gs)
    return (vals * scales.to(torch.float32).unsqueeze(-1)).view(out_f, in_f).to(dtype)


def _pack_last_axis(codes: torch.Tensor) -> torch.Tensor:
    """Pack 8 nibbles along the last axis into int32 (bit pattern of the uint32)."""
    *lead, n = codes.shape
    assert n % 8 == 0
    c = codes.to(torch.int64).view(*lead, n // 8, 8)
    shifts = torch.arange(8, device=codes.device, dtype=torch.int64) * 4
    word = (c << shifts).sum(dim=-1)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
    return word.to(torch.int32)


def _unpack_last_axis(packed: torch.Tensor) -> torch.Tensor:
    p = packed.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(8, device=packed.device, dtype=torch.int64) * 4
    nib = (p.unsqueeze(-1) >> shifts) & 0xF
    return nib.reshape(*packed.shape[:-1], packed.shape[-1] * 8).to(torch.uint8)


def pack_mmfp4(codes: torch.Tensor, scales: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """codes ``[out, in]`` -> packed ``int32 [out, in/8]``, scales ``fp16 [out, in/gs]``."""
    return _pack_last_axis(codes), scales.to(torch.float16).contiguous()


def pack_marlin_fp4(codes: torch.Tensor, scales: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """codes ``[out, in]`` -> packed ``int32 [in/8, out]``, scales ``fp16 [in/gs, out]``."""
    return _pack_last_axis(codes).t().contiguous(), scales.to(torch.float16).t().contiguous()


def unpack_mmfp4(packed: torch.Tensor, scales: torch.Tensor, in_features: Optional[int] = None
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Inverse of :func:`pack_mmfp4`.  Accepts scales as ``[out, n_groups]`` or ``[n_groups, out]``
    and stacked banks ``[E, out, in/8]``; returns codes ``[.., out, in]`` and scales ``[.., out, n_groups]``."""
    out_f = packed.shape[-2]
    codes = _unpack_last_axis(packed)
    if in_features is not None:
        codes = codes[..., :in_features]
    if scales.shape[-2] != out_f and scales.shape[-1] == out_f:
        scales = scales.transpose(-1, -2)
    elif scales.shape[-2] == out_f and scales.shape[-1] == out_f:
        pass  # square and ambiguous: the row-packed writers emit [out, n_groups]
    return codes, scales.contiguous()


def unpack_marlin_fp4(packed: torch.Tensor, scales: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Inverse of :func:`pack_marlin_fp4`; returns codes ``[out, in]``, scales ``[out, n_groups]``."""
    codes = _unpack_last_axis(packed.t().contiguous())
    return codes, scales.t().contiguous()


def quantize_fp4(w: torch.Tensor, group_size: int = 128, layout: str = "marlin_fp4"):
    """One-call RTN quantizer returning tensors in a checkpoint layout."""
    gs = pick_group_size(w.shape[1], group_size)
    if w.is_cuda and w.dim() == 2 and layout in ("marlin_fp4", "mmfp4"):
        from .. import ops                      # one fused quantize + pack launch on the GPU, same bits
        packed, scales = ops.fp4_quantize_pack(w, gs)
        return (packed, scales, gs) if layout == "mmfp4" else (packed.t().contiguous(), scales.t().contiguous(), gs)
    codes, scales = quantize_codes(w, gs)
    if layout == "marlin_fp4":
        return (*pack_marlin_fp4(codes, scales), gs)
    if layout == "mmfp4":
        return (*pack_mmfp4(codes, scales), gs)
    raise ValueError(layout)


# ---------------------------------------------------------------------------------------------
# Device tile layout
# ---------------------------------------------------------------------------------------------
TILE_ROWS = 16
TILE_K = 64


def padded_dims(out_f: int, in_f: int) -> Tuple[int, int]:
    return (out_f + TILE_ROWS - 1) // TILE_ROWS * TILE_ROWS, (in_f + TILE_K - 1) // TILE_K * TILE_K


def to_tile_layout(codes: torch.Tensor, scales: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """codes ``uint8 [out, in]`` + scales ``[out, n_groups]`` -> device tile layout.

    Returns ``(qtile int32 [out_p/16, in_p/64, 32, 4], stile fp16 [out_p/16, n_groups_p, 8, 2], gs)``.
    Rows are padded to 16 and columns to 64 with zero codes; padded groups get scale 0."""
    out_f, in_f = codes.shape
    n_groups = scales.shape[1]
    gs = in_f // n_groups
    assert gs * n_groups == in_f and gs % 16 == 0, "group size must be a multiple of 16 for the tile layout"
    out_p, in_p = padded_dims(out_f, in_f)
    if in_p != in_f:
        assert in_p % gs == 0 or gs % 64 == 0 or 64 % gs == 0
    ng_p = (in_p + gs - 1) // gs
    if (out_p, in_p) != (out_f, in_f):
        c = torch.zeros(out_p, in_p, dtype=torch.uint8, device=codes.device)
        c[:out_f, :in_f] = codes
        codes = c
    s = torch.zeros(out_p, ng_p, dtype=torch.float16, device=scales.device)
    s[:out_f, :n_groups] = scales.to(torch.float16)
    # n = rt*16 + h*8 + g ;  k = kc*64 + ks*16 + kh*8 + t*2 + e
    c = codes.view(out_p // 16, 2, 8, in_p // 64, 4, 2, 4, 2).to(torch.int64)
    # axes:         rt       h  g   kc        ks kh t  e
    h = torch.arange(2, device=codes.device).view(1, 2, 1, 1, 1, 1, 1, 1)
    kh = torch.arange(2, device=codes.device).view(1, 1, 1, 1, 1, 2, 1, 1)
    e = torch.arange(2, device=codes.device).view(1, 1, 1, 1, 1, 1, 1, 2)
    j = h + 2 * kh                                           # fragment register of the element
    word = (((c >> 3) << (16 * e + 15 - j)) + ((c & 7) << (16 * e + 9 - 3 * j))).sum(dim=(1, 5, 7))     # [rt, g, kc, ks, t]
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)
    qtile = word.permute(0, 2, 1, 4, 3).contiguous().view(out_p // 16, in_p // 64, 32, 4)
    stile = s.view(out_p // 16, 2, 8, ng_p).permute(0, 3, 2, 1).contiguous()   # [rt, grp, g, h]
    return qtile, stile, gs


def from_tile_layout(qtile: torch.Tensor, stile: torch.Tensor, out_f: int, in_f: int, group_size: int
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Inverse of :func:`to_tile_layout` (used by tests and by the CPU fallback)."""
    n_rt, n_kc = qtile.shape[0], qtile.shape[1]
    w = (qtile.to(torch.int64) & 0xFFFFFFFF).view(n_rt, n_kc, 8, 4, 4)       # [rt, kc, g, t, ks]
    dev = qtile.device
    h = torch.arange(2, device=dev).view(2, 1, 1)
    kh = torch.arange(2, device=dev).view(1, 2, 1)
    e = torch.arange(2, device=dev).view(1, 1, 2)
    j = h + 2 * kh                                                             # [h, kh, 1]
    w8 = w.view(n_rt, n_kc, 8, 4, 4, 1, 1, 1)
    nib = (((w8 >> (16 * e + 15 - j)) & 1) << 3) | ((w8 >> (16 * e + 9 - 3 * j)) & 7)      # [rt,kc,g,t,ks,h,kh,e]
    codes = nib.permute(0, 5, 2, 1, 4, 6, 3, 7).contiguous().view(n_rt * 16, n_kc * 64).to(torch.uint8)
    ng = stile.shape[1]
    scales = stile.permute(0, 3, 2, 1).contiguous().view(n_rt * 16, ng)
    n_groups = in_f // group_size
    return codes[:out_f, :in_f], scales[:out_f, :n_groups]


def e2m1_value(code: int) -> float:
    return E2M1_VALUES[code & 0xF]


def numpy_unpack_fp4(packed: np.ndarray) -> np.ndarray:
    """NumPy nibble unpack along the last axis (LSB nibble first)."""
    p = packed.astype(np.uint32)
    shifts = (np.arange(8, dtype=np.uint32) * 4)
    return ((p[..., None] >> shifts) & 0xF).reshape(*p.shape[:-1], p.shape[-1] * 8).astype(np.uint8)
