"""Round-to-nearest group quantizers and packers for every weight format the engine reads.

Formats: ``fp4`` (E2M1), ``int4`` (unsigned with zero point, or symmetric), ``nf4``,
``int8``, ``fp8`` (E4M3 / E5M2), ``int3``, ``int2``, ``nf3``, ``nf2``.

Parity: reference ``metal_marlin/quantize.py:112`` (``pack_fp4_weights``),
``metal_marlin/quantize_fp4.py:131``, ``metal_marlin/sub4bit.py`` and
``metal_marlin/fp8_utils.py``.  All quantizers return *codes* plus per-group
parameters; packers turn codes into the little-endian, LSB-first bit streams the
checkpoint formats use.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .._compat import NF4_VALUES
from ..formats import fp4 as fp4fmt

NF3_VALUES = (-1.0, -0.5350227355957031, -0.2469314038753510, 0.0,
              0.1833375245332718, 0.3819939494132996, 0.6229856610298157, 1.0)
NF2_VALUES = (-1.0, -0.3333333, 0.3333333, 1.0)


@dataclass
class QuantizedTensor:
    """Codes plus parameters in the canonical ``[out, in]`` orientation."""
    codes: torch.Tensor                 # uint8 [out, in]
    scales: torch.Tensor                # [out, n_groups]
    zeros: Optional[torch.Tensor]       # [out, n_groups] or None
    fmt: str
    group_size: int
    bits: int

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        return dequantize(self, dtype)


def _grouped(w: torch.Tensor, gs: int) -> torch.Tensor:
    out_f, in_f = w.shape
    assert in_f % gs == 0, (in_f, gs)
    return w.detach().to(torch.float32).view(out_f, in_f // gs, gs)


def quantize_fp4(w: torch.Tensor, group_size: int = 128) -> QuantizedTensor:
    codes, scales = fp4fmt.quantize_codes(w, group_size)
    return QuantizedTensor(codes, scales, None, "fp4", group_size, 4)


def _nearest_codebook(x: torch.Tensor, book: torch.Tensor) -> torch.Tensor:
    mids = (book[1:] + book[:-1]) / 2
    return torch.bucketize(x, mids)


def quantize_codebook(w: torch.Tensor, values, fmt: str, bits: int, group_size: int) -> QuantizedTensor:
    g = _grouped(w, group_size)
    absmax = g.abs().amax(dim=-1, keepdim=True).clamp_min(1e-8)
    book = torch.tensor(values, dtype=torch.float32, device=w.device)
    codes = _nearest_codebook(g / absmax, book).to(torch.uint8).view_as(w)
    return QuantizedTensor(codes, absmax.squeeze(-1).to(torch.float16), None, fmt, group_size, bits)


def quantize_nf4(w, group_size=64):
    return quantize_codebook(w, NF4_VALUES, "nf4", 4, group_size)


def quantize_nf3(w, group_size=64):
    return quantize_codebook(w, NF3_VALUES, "nf3", 3, group_size)


def quantize_nf2(w, group_size=64):
    return quantize_codebook(w, NF2_VALUES, "nf2", 2, group_size)


def quantize_uint(w: torch.Tensor, bits: int, group_size: int = 128, symmetric: bool = False) -> QuantizedTensor:
    """Affine (zero-point) or symmetric integer quantization with ``2**bits`` levels."""
    g = _grouped(w, group_size)
    qmax = 2 ** bits - 1
    if symmetric:
        absmax = g.abs().amax(dim=-1, keepdim=True).clamp_min(1e-8)
        half = (qmax + 1) // 2
        scale = absmax / (half - 1 if half > 1 else 1)
        zero = torch.full_like(scale, float(half))
    else:
        lo = g.amin(dim=-1, keepdim=True)
        hi = g.amax(dim=-1, keepdim=True)
        scale = ((hi - lo) / qmax).clamp_min(1e-8)
        zero = (-lo / scale).round().clamp_(0, qmax)
    codes = (g / scale + zero).round().clamp_(0, qmax).to(torch.uint8).view_as(w)
    return QuantizedTensor(codes, scale.squeeze(-1).to(torch.float16), zero.squeeze(-1).to(torch.float16),
                           f"int{bits}", group_size, bits)


def quantize_int4(w, group_size=128, symmetric=False):
    return quantize_uint(w, 4, group_size, symmetric)


def quantize_int3(w, group_size=64):
    return quantize_uint(w, 3, group_size)


def quantize_int2(w, group_size=64):
    return quantize_uint(w, 2, group_size)


def quantize_int8(w: torch.Tensor, group_size: int = 128) -> QuantizedTensor:
    g = _grouped(w, group_size)
    scale = (g.abs().amax(dim=-1, keepdim=True) / 127.0).clamp_min(1e-8)
    q = (g / scale).round().clamp_(-127, 127)
    codes = (q + 128).to(torch.uint8).view_as(w)
    zero = torch.full_like(scale, 128.0)
    return QuantizedTensor(codes, scale.squeeze(-1).to(torch.float16), zero.squeeze(-1).to(torch.float16),
                           "int8", group_size, 8)


def quantize_fp8(w: torch.Tensor, group_size: int = 128, variant: str = "e4m3") -> QuantizedTensor:
    g = _grouped(w, group_size)
    fdt = torch.float8_e4m3fn if variant == "e4m3" else torch.float8_e5m2
    fmax = 448.0 if variant == "e4m3" else 57344.0
    scale = (g.abs().amax(dim=-1, keepdim=True) / fmax).clamp_min(1e-12)
    q = (g / scale).clamp_(-fmax, fmax).to(fdt)
    codes = q.view(torch.uint8).view_as(w)
    return QuantizedTensor(codes, scale.squeeze(-1).to(torch.float32), None, f"fp8_{variant}", group_size, 8)


def dequantize(q: QuantizedTensor, dtype=torch.float32) -> torch.Tensor:
    out_f, in_f = q.codes.shape
    ng = q.scales.shape[1]
    gs = in_f // ng
    sc = q.scales.to(torch.float32).unsqueeze(-1)
    c = q.codes.view(out_f, ng, gs)
    if q.fmt == "fp4":
        return fp4fmt.dequantize_codes(q.codes, q.scales, dtype)
    if q.fmt in ("nf4", "nf3", "nf2"):
        book = torch.tensor({"nf4": NF4_VALUES, "nf3": NF3_VALUES, "nf2": NF2_VALUES}[q.fmt],
                            dtype=torch.float32, device=q.codes.device)
        return (book[c.long()] * sc).view(out_f, in_f).to(dtype)
    if q.fmt.startswith("int"):
        z = q.zeros.to(torch.float32).unsqueeze(-1)
        return ((c.to(torch.float32) - z) * sc).view(out_f, in_f).to(dtype)
    if q.fmt.startswith("fp8"):
        fdt = torch.float8_e4m3fn if q.fmt.endswith("e4m3") else torch.float8_e5m2
        return (c.contiguous().view(fdt).to(torch.float32) * sc).view(out_f, in_f).to(dtype)
    raise ValueError(q.fmt)


QUANTIZERS = {
    "fp4": quantize_fp4, "int4": quantize_int4, "nf4": quantize_nf4, "int8": quantize_int8,
    "fp8": quantize_fp8, "int3": quantize_int3, "int2": quantize_int2, "nf3": quantize_nf3, "nf2": quantize_nf2,
}


def quantize(w: torch.Tensor, fmt: str = "fp4", group_size: int = 128) -> QuantizedTensor:
    return QUANTIZERS[fmt](w, group_size)


# ---------------------------------------------------------------------------------------------
# Bit-stream packing (LSB first, little endian) for arbitrary bit widths 1..8
# ---------------------------------------------------------------------------------------------
def pack_bits(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """Pack the last axis of ``codes`` (values < 2**bits) into bytes, LSB first."""
    *lead, n = codes.shape
    assert (n * bits) % 8 == 0, "row must fill whole bytes"
    c = codes.to(torch.int64).reshape(-1, n)
    bitpos = torch.arange(bits, device=codes.device)
    stream = ((c.unsqueeze(-1) >> bitpos) & 1).reshape(c.shape[0], n * bits)
    stream = stream.view(c.shape[0], n * bits // 8, 8)
    w = (stream << torch.arange(8, device=codes.device)).sum(-1)
    return w.to(torch.uint8).view(*lead, n * bits // 8)


def unpack_bits(packed: torch.Tensor, bits: int, n: int) -> torch.Tensor:
    *lead, nb = packed.shape
    p = packed.to(torch.int64).reshape(-1, nb)
    stream = ((p.unsqueeze(-1) >> torch.arange(8, device=packed.device)) & 1).reshape(p.shape[0], nb * 8)
    stream = stream[:, : n * bits].reshape(p.shape[0], n, bits)
    c = (stream << torch.arange(bits, device=packed.device)).sum(-1)
    return c.to(torch.uint8).view(*lead, n)


def quantization_error(w: torch.Tensor, q: QuantizedTensor) -> Tuple[float, float]:
    """(relative Frobenius error, max abs error)."""
    d = dequantize(q) - w.to(torch.float32)
    return float(d.norm() / w.to(torch.float32).norm().clamp_min(1e-12)), float(d.abs().max())
