"""Linear layers over quantized weights.

* ``MMFP4Linear`` - FP4 (E2M1) weights in the device tile layout; the layer the reference calls
  ``MMFP4Linear`` (``metal_marlin/layers/mmfp4_linear.py:600``): accepts packed ``uint32 [out, in/8]`` + scales in
  either orientation, optional bias and fused activation.  Where the reference multiplies by a cached fp16
  de-quantized copy for M <= 16, this layer streams the FP4 bytes (``csrc/gemv.cu``) and uses the tcgen05 GEMM above.
* ``QuantizedLinear`` - INT8 / INT4 / INT3 / INT2 / FP8 / NF4 / NF3 / NF2 group formats through one codebook GEMV
  (``csrc/quant_gemv.cu``); large M de-quantizes once and runs a bf16 GEMM.
* ``TrellisLinear`` - 2-8 bit trellis weights (``metal_marlin/trellis/linear.py:50,533``): decode reads the tile bit
  stream directly (``csrc/trellis.cu``), prefill de-quantizes to bf16 and runs the bf16 tcgen05 GEMM.
* ``HadamardLinear`` - wraps a layer whose weight was quantized in a block-Hadamard-rotated basis (MR-GPTQ).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .. import ops
from ..formats import trellis as trfmt
from ..ops.weights import FP4Weight
from ..quant import rtn
from .lora import LoRAMixin

DECODE_MAX_M = 8


def _bf16_matmul(x2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x2 [M, K] @ w [N, K]^T`` in bf16: the tcgen05 GEMM when K fits its 64-wide K tiles, a library GEMM otherwise."""
    if x2.is_cuda and x2.shape[1] % 64 == 0 and x2.stride(0) % 8 == 0:
        return ops.bf16_gemm(x2, w)
    if x2.is_cuda:
        return torch.matmul(x2, w.t())
    return (x2.float() @ w.float().t()).to(torch.bfloat16)


class MMFP4Linear(LoRAMixin):
    def __init__(self, weight: FP4Weight, bias: Optional[torch.Tensor] = None, activation: Optional[str] = None):
        self.weight, self.bias, self.activation = weight, bias, activation
        self.in_features, self.out_features = weight.in_features, weight.out_features

    @classmethod
    def from_pretrained_weight(cls, packed: torch.Tensor, scales: torch.Tensor, bias=None, device=None, layout: str = "mmfp4"):
        w = FP4Weight.from_marlin_fp4(packed, scales, device) if layout == "marlin_fp4" else FP4Weight.from_mmfp4(packed, scales, device)
        return cls(w, None if bias is None else bias.to(w.device, torch.bfloat16))

    @classmethod
    def from_float(cls, w: torch.Tensor, group_size: int = 128, bias=None, device=None):
        return cls(FP4Weight.from_float(w, group_size, device), bias)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        y = ops.linear(x.reshape(-1, shape[-1]).to(torch.bfloat16), self.weight, bias=self.bias)
        if self.activation == "silu":
            y = F.silu(y)
        elif self.activation == "gelu":
            y = F.gelu(y)
        return y.view(*shape[:-1], self.out_features)

    forward = __call__

    def dequantize(self, dtype=torch.bfloat16) -> torch.Tensor:
        return self.weight.dequantize(dtype)


def _lut_for(fmt: str, device) -> torch.Tensor:
    lut = torch.zeros(256, dtype=torch.float32)
    if fmt.startswith("int"):
        lut = torch.arange(256, dtype=torch.float32)
    elif fmt.startswith("fp8"):
        dt = torch.float8_e5m2 if fmt.endswith("e5m2") else torch.float8_e4m3fn
        lut = torch.arange(256, dtype=torch.uint8).view(dt).to(torch.float32)
        lut = torch.nan_to_num(lut, nan=0.0, posinf=0.0, neginf=0.0)
    else:
        book = {"nf4": rtn.NF4_VALUES, "nf3": rtn.NF3_VALUES, "nf2": rtn.NF2_VALUES}[fmt]
        lut[: len(book)] = torch.tensor(book, dtype=torch.float32)
    return lut.to(device)


class QuantizedLinear(LoRAMixin):
    """Group-quantized linear for the non-FP4 formats."""
    is_generic = True
    names = None

    def __init__(self, q: rtn.QuantizedTensor, bias: Optional[torch.Tensor] = None, device=None):
        device = torch.device(device) if device is not None else q.codes.device
        self.fmt, self.group_size = q.fmt, q.group_size
        self.out_features, self.in_features = q.codes.shape
        self.dev_bits = {1: 2, 2: 2, 3: 4, 4: 4}.get(q.bits, 8)          # 3-bit codes are held as 4-bit on the device
        per = 8 // self.dev_bits
        c = q.codes.to(device).long()
        if self.in_features % per:
            raise ValueError("in_features must be a multiple of the codes-per-byte of the format")
        sh = torch.arange(per, device=device) * self.dev_bits
        self.codes = (c.view(self.out_features, -1, per) << sh).sum(-1).to(torch.uint8).contiguous()
        self.scales = q.scales.to(device, torch.float16).contiguous()
        self.zeros = None if q.zeros is None else q.zeros.to(device, torch.float16).contiguous()
        self.lut = _lut_for(q.fmt, device)
        self.bias = None if bias is None else bias.to(device, torch.bfloat16)
        self._deq = None

    @classmethod
    def from_float(cls, w: torch.Tensor, fmt: str = "int4", group_size: int = 128, bias=None, device=None):
        return cls(rtn.quantize(w.to(torch.float32), fmt, group_size), bias, device)

    def dequantize(self, dtype=torch.bfloat16) -> torch.Tensor:
        from ..ops import reference as ref
        return ref.codebook_dequant(self.codes, self.scales, self.zeros, self.lut, self.in_features, self.group_size, self.dev_bits).to(dtype)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(torch.bfloat16)
        cpl = 16 * (8 // self.dev_bits)
        fast = x2.shape[0] <= DECODE_MAX_M and self.in_features % cpl == 0 and self.group_size % cpl == 0
        if fast:
            y = ops.codebook_gemv(x2.contiguous(), self.codes, self.scales, self.zeros, self.lut, self.in_features, self.group_size,
                                  self.dev_bits)
        elif ops.codebook_gemm_ok(x2, self.in_features, self.group_size, self.dev_bits):
            # more than a few rows: the same codes on the tensor cores, expanded inside the GEMM's main loop
            y = ops.codebook_gemm(x2.contiguous(), self.codes, self.scales, self.zeros, self.lut, self.in_features, self.group_size,
                                  self.dev_bits)
        else:
            if self._deq is None:
                self._deq = self.dequantize(torch.bfloat16)
            y = _bf16_matmul(x2.contiguous(), self._deq)
        if self.bias is not None:
            y = y + self.bias
        return y.view(*shape[:-1], self.out_features)

    forward = __call__


class Sparse24Linear(LoRAMixin):
    """2:4 structured-sparse FP4 linear: of every four consecutive input columns the two of largest magnitude are kept,
    quantized to E2M1 with one fp16 scale per ``group_size`` dense columns, and stored with a 4-bit position word per group -
    0.375 bytes per dense weight (FP4 dense: 0.5).  The product runs on the tensor-core GEMM, which scatters the kept values
    into a dense tile inside its main loop (``csrc/gemm_sm100.cu``, weight format 4); no dense copy of the matrix exists.

    Parity: reference ``src/sparse_gemm.metal:334`` (``marlin_gemm_sparse_fp4``: compressed FP4 values + 2-bit position
    metadata, dense tile rebuilt by the loader), ``src/sparse.metal:630``, ``metal_marlin/prune_weights.py`` (magnitude 2:4)."""
    is_generic = True
    names = None

    def __init__(self, codes, meta, scales, out_features: int, in_features: int, group_size: int, bias=None):
        self.codes, self.meta, self.scales = codes, meta, scales
        self.out_features, self.in_features, self.group_size = out_features, in_features, group_size
        self.bias = bias

    @staticmethod
    def prune(w: torch.Tensor):
        """``(kept values [out, in / 4, 2], positions [out, in / 4, 2] ascending)`` of the magnitude 2:4 pattern."""
        out_f, in_f = w.shape
        g = w.reshape(out_f, in_f // 4, 4)
        pos = g.abs().topk(2, -1).indices.sort(-1).values
        return g.gather(-1, pos), pos

    @classmethod
    def from_float(cls, w: torch.Tensor, group_size: int = 128, bias=None, device=None):
        from ..formats import fp4 as fp4fmt
        out_f, in_f = w.shape
        if in_f % 64 or in_f % group_size or group_size < 32 or group_size & (group_size - 1):
            raise ValueError("in_features must be a multiple of 64 and of the group size (a power of two >= 32)")
        device = torch.device(device) if device is not None else w.device
        vals, pos = cls.prune(w.to(torch.float32))
        # the kept values of a dense group of `group_size` columns are `group_size / 2` consecutive compact columns
        codes, scales = fp4fmt.quantize_codes(vals.reshape(out_f, in_f // 2), group_size // 2)
        c = codes.view(out_f, in_f // 4, 2)
        packed = (c[..., 0] | (c[..., 1] << 4)).to(torch.uint8)
        nib = (pos[..., 0] | (pos[..., 1] << 2)).to(torch.uint8).view(out_f, in_f // 8, 2)
        meta = (nib[..., 0] | (nib[..., 1] << 4)).to(torch.uint8)
        b = None if bias is None else bias.to(device, torch.bfloat16)
        return cls(packed.contiguous().to(device), meta.contiguous().to(device), scales.contiguous().to(device), out_f, in_f, group_size, b)

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        from ..ops import reference as ref
        return ref.sparse24_dequant(self.codes, self.meta, self.scales, self.in_features, self.group_size).to(dtype)

    def nbytes(self) -> int:
        return self.codes.numel() + self.meta.numel() + self.scales.numel() * 2

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(torch.bfloat16)
        y = ops.sparse24_gemm(x2, self.codes, self.meta, self.scales, self.in_features, self.group_size)
        if self.bias is not None:
            y = y + self.bias
        return y.view(*shape[:-1], self.out_features)

    forward = __call__


class TrellisLinear(LoRAMixin):
    is_generic = True
    names = None

    def __init__(self, tw: trfmt.TrellisWeight, device=None, bias: Optional[torch.Tensor] = None):
        device = torch.device(device) if device is not None else tw.indices.device
        self.out_features, self.in_features = tw.shape
        self.bits, self.group_size = tw.bits, tw.group_size
        su, sv = tw.su.float(), tw.sv.float()
        if su.numel() == self.out_features and sv.numel() == self.in_features and self.out_features != self.in_features:
            su, sv = sv, su
        self.codes = tw.indices.reshape(-1)[1:].contiguous().to(device)
        self.scales = tw.scales.float().contiguous().to(device)
        self.su, self.sv = su.contiguous().to(device), sv.contiguous().to(device)
        if self.codes.data_ptr() % 16:       # the code stream starts one byte into its checkpoint tensor: the kernels read aligned words
            self.codes = self.codes.clone()
        self.bias = None if bias is None else bias.to(device, torch.bfloat16)
        self.device = device
        self._deq = None
        self._desc = None

    @classmethod
    def from_float(cls, w: torch.Tensor, bits: int = 4, group_size: int = 128, device=None):
        return cls(trfmt.quantize_trellis(w, bits, group_size), device)

    @classmethod
    def random(cls, out_f: int, in_f: int, bits: int = 4, group_size: int = 128, device="cpu", seed: int = 0, std: float = 0.02):
        """Random-init matrix drawn directly in the quantized domain (uniform codes, one scale per group and row sized so
        that the weights have about ``std`` spread): synthetic benchmark models of tens of billions of parameters are built
        in seconds, without ever holding a float copy."""
        self = cls.__new__(cls)
        dev = torch.device(device)
        g = torch.Generator(device=dev).manual_seed(seed)
        self.out_features, self.in_features, self.bits, self.group_size = out_f, in_f, bits, group_size
        n_tiles = ((out_f + 15) // 16) * ((in_f + 15) // 16)
        self.codes = torch.randint(0, 256, (n_tiles * 32 * bits,), dtype=torch.uint8, device=dev, generator=g)
        levels = (1 << bits) - 1
        # uniform codes have a spread of about levels / sqrt(12) grid steps
        step = std / (max(levels, 1) / 3.4641 * 1.24371088)
        self.scales = torch.full(((in_f + group_size - 1) // group_size, out_f), step, dtype=torch.float32, device=dev)
        self.su = (torch.randint(0, 2, (in_f,), device=dev, generator=g).float() * 2 - 1).contiguous()
        self.sv = (torch.randint(0, 2, (out_f,), device=dev, generator=g).float() * 2 - 1).contiguous()
        self.bias, self.device, self._deq, self._desc = None, dev, None, None
        return self

    def dequantize(self, dtype=torch.bfloat16) -> torch.Tensor:
        return ops.trellis_dequant(self.codes, self.scales, self.su, self.sv, self.out_features, self.in_features, self.bits,
                                   self.group_size).to(dtype)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(torch.bfloat16).contiguous()
        if x2.shape[0] <= DECODE_MAX_M:
            y = ops.trellis_gemv(x2, self.codes, self.scales, self.su, self.sv, self.out_features, self.bits, self.group_size)
        elif ops.trellis_gemm_ok(x2, self.in_features, self.group_size):
            # tensor cores: the codes are decoded inside the GEMM's main loop, no bf16 copy of the matrix exists
            if self._desc is None:
                self._desc = torch.tensor([ops.trellis_desc_row(self.codes, self.scales, self.su, self.sv, self.out_features,
                                                                self.in_features, self.bits, self.group_size)],
                                          dtype=torch.int64).to(x2.device)
            y = ops.trellis_gemm(x2, self._desc, self.out_features, self.in_features)
        else:
            w = self.dequantize(torch.bfloat16)          # transient: the bf16 copy is not kept between calls
            y = _bf16_matmul(x2, w)
        if self.bias is not None:
            y = y + self.bias
        return y.view(*shape[:-1], self.out_features)

    forward = __call__

    def nbytes(self) -> int:
        return self.codes.numel() + 4 * (self.scales.numel() + self.su.numel() + self.sv.numel())


class HadamardLinear(LoRAMixin):
    """``y = inner(block_hadamard(x))`` for a weight stored in the rotated basis."""
    is_generic = True
    names = None

    def __init__(self, inner, block: int = 128):
        self.inner, self.block = inner, block
        self.in_features, self.out_features = inner.in_features, inner.out_features

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.inner(ops.hadamard(x.to(torch.bfloat16).contiguous() if x.is_cuda else x, self.block))

    forward = __call__
