"""Device-resident quantized weight containers.

``FP4Weight`` / ``FP4ExpertBank`` hold a matrix (or a stacked bank of expert
matrices) in the device tile layout the sm_100a kernels read (see
``formats/fp4.py``).  They are built once at load time from any checkpoint
layout — the "repack at load" step; the checkpoint bytes themselves are never
changed.  Parity: reference ``metal_marlin/layers/mmfp4_linear.py:414``
(``_rowpacked_to_gpu_layout``) and ``metal_marlin/glm4_moe_experts.py:140-215``
(stacked expert buffers).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..formats import fp4 as fp4fmt


class FP4Weight:
    __slots__ = ("qtile", "stile", "out_features", "in_features", "group_size", "_deq", "names", "hadamard_block")

    def __init__(self, qtile, stile, out_features, in_features, group_size, hadamard_block: int = 0):
        self.qtile = qtile
        self.stile = stile
        self.out_features = int(out_features)
        self.in_features = int(in_features)
        self.group_size = int(group_size)
        self._deq = None
        self.names = None            # [(checkpoint tensor name, rows)] when loaded from a checkpoint (calibration hooks)
        # > 0: the matrix is stored in a block-Hadamard-rotated input basis (MR-GPTQ); consumers rotate the activation
        self.hadamard_block = int(hadamard_block)

    # ------------------------------------------------------------------ constructors
    @classmethod
    def from_codes(cls, codes: torch.Tensor, scales: torch.Tensor, device=None) -> "FP4Weight":
        out_f, in_f = codes.shape
        if device is not None:
            codes, scales = codes.to(device), scales.to(device)
        qtile, stile, gs = fp4fmt.to_tile_layout(codes, scales)
        return cls(qtile, stile, out_f, in_f, gs)

    @classmethod
    def from_float(cls, w: torch.Tensor, group_size: int = 128, device=None) -> "FP4Weight":
        gs = fp4fmt.pick_group_size(w.shape[1], group_size)
        if device is not None:
            w = w.to(device)
        codes, scales = fp4fmt.quantize_codes(w, gs)
        return cls.from_codes(codes, scales)

    @classmethod
    def from_mmfp4(cls, packed: torch.Tensor, scales: torch.Tensor, device=None) -> "FP4Weight":
        if device is not None:
            packed, scales = packed.to(device), scales.to(device)
        codes, sc = fp4fmt.unpack_mmfp4(packed, scales)
        return cls.from_codes(codes, sc)

    @classmethod
    def from_marlin_fp4(cls, packed: torch.Tensor, scales: torch.Tensor, device=None) -> "FP4Weight":
        if device is not None:
            packed, scales = packed.to(device), scales.to(device)
        codes, sc = fp4fmt.unpack_marlin_fp4(packed, scales)
        return cls.from_codes(codes, sc)

    @classmethod
    def concat_rows(cls, parts: Sequence["FP4Weight"]) -> "FP4Weight":
        """Stack matrices that share the input dimension along the output axis
        (fused q_a|kv_a, q|k|v, gate|up).  Each part must have a multiple of 16 rows."""
        p0 = parts[0]
        for p in parts:
            assert p.in_features == p0.in_features and p.group_size == p0.group_size
            assert p.out_features % 16 == 0, "row-concat needs 16-row aligned parts"
        q = torch.cat([p.qtile for p in parts], 0)
        s = torch.cat([p.stile for p in parts], 0)
        assert len({p.hadamard_block for p in parts}) == 1, "row-concatenated matrices must share one input rotation"
        w = cls(q, s, sum(p.out_features for p in parts), p0.in_features, p0.group_size, p0.hadamard_block)
        if all(p.names for p in parts):
            w.names = [n for p in parts for n in p.names]
        return w

    # ------------------------------------------------------------------ tensor-parallel shards
    def slice_rows(self, r0: int, r1: int) -> "FP4Weight":
        """Output rows ``[r0, r1)`` (column-parallel shard); bounds must be multiples of 16."""
        assert r0 % 16 == 0 and (r1 % 16 == 0 or r1 == self.out_features)
        return FP4Weight(self.qtile[r0 // 16: (r1 + 15) // 16].contiguous(), self.stile[r0 // 16: (r1 + 15) // 16].contiguous(),
                         r1 - r0, self.in_features, self.group_size, self.hadamard_block)

    def slice_cols(self, k0: int, k1: int) -> "FP4Weight":
        """Input columns ``[k0, k1)`` (row-parallel shard); bounds must be multiples of max(64, group size)."""
        unit = max(64, self.group_size)
        assert k0 % unit == 0 and (k1 % unit == 0 or k1 == self.in_features), (k0, k1, unit)
        gs = self.group_size
        hb = self.hadamard_block
        assert not hb or (k0 % hb == 0 and (k1 - k0) % hb == 0), "a column shard must not cut a rotation block"
        return FP4Weight(self.qtile[:, k0 // 64: (k1 + 63) // 64].contiguous(),
                         self.stile[:, k0 // gs: (k1 + gs - 1) // gs].contiguous(), self.out_features, k1 - k0, gs, hb)

    # ------------------------------------------------------------------ views
    @property
    def device(self):
        return self.qtile.device

    @property
    def padded_in(self) -> int:
        return self.qtile.shape[1] * 64

    def to(self, device) -> "FP4Weight":
        return FP4Weight(self.qtile.to(device), self.stile.to(device), self.out_features, self.in_features,
                         self.group_size, self.hadamard_block)

    def codes_scales(self):
        return fp4fmt.from_tile_layout(self.qtile, self.stile, self.out_features, self.in_features, self.group_size)

    def dequantize(self, dtype=torch.float32, cache: bool = False) -> torch.Tensor:
        if self._deq is not None and self._deq.dtype == dtype:
            return self._deq
        codes, scales = self.codes_scales()
        w = fp4fmt.dequantize_codes(codes, scales, dtype)
        if cache:
            self._deq = w
        return w

    def nbytes(self) -> int:
        return self.qtile.numel() * 4 + self.stile.numel() * 2


class FP4ExpertBank:
    """``E`` (+ shared) expert matrices of identical shape stacked on a leading axis."""
    __slots__ = ("qtile", "stile", "num_experts", "out_features", "in_features", "group_size", "_deq", "names", "hadamard_block")

    def __init__(self, qtile, stile, out_features, in_features, group_size, hadamard_block: int = 0):
        self.hadamard_block = int(hadamard_block)      # shared input rotation of every expert (0 = none)
        self.qtile = qtile            # [E, N/16, K/64, 32, 4] int32
        self.stile = stile            # [E, N/16, K/gs, 8, 2] fp16
        self.num_experts = qtile.shape[0]
        self.out_features = int(out_features)
        self.in_features = int(in_features)
        self.group_size = int(group_size)
        self._deq = None
        self.names = None            # per expert: [(checkpoint tensor name, rows)] when loaded from a checkpoint

    @classmethod
    def from_weights(cls, ws: List[FP4Weight]) -> "FP4ExpertBank":
        w0 = ws[0]
        bank = cls(torch.stack([w.qtile for w in ws]), torch.stack([w.stile for w in ws]),
                   w0.out_features, w0.in_features, w0.group_size)
        if any(w.names for w in ws):
            bank.names = [w.names or [] for w in ws]
        return bank

    @classmethod
    def from_float(cls, w: torch.Tensor, group_size: int = 128) -> "FP4ExpertBank":
        """``w [E, out, in]`` float -> quantized bank, one expert at a time (bounded memory)."""
        return cls.from_weights([FP4Weight.from_float(w[e], group_size) for e in range(w.shape[0])])

    @property
    def device(self):
        return self.qtile.device

    def slice_rows(self, ranges) -> "FP4ExpertBank":
        """Keep the output-row ranges ``[(r0, r1), ...]`` (multiples of 16) of every expert, concatenated."""
        q = torch.cat([self.qtile[:, r0 // 16: r1 // 16] for r0, r1 in ranges], 1).contiguous()
        s = torch.cat([self.stile[:, r0 // 16: r1 // 16] for r0, r1 in ranges], 1).contiguous()
        return FP4ExpertBank(q, s, sum(r1 - r0 for r0, r1 in ranges), self.in_features, self.group_size, self.hadamard_block)

    def slice_cols(self, k0: int, k1: int) -> "FP4ExpertBank":
        unit = max(64, self.group_size)
        assert k0 % unit == 0 and (k1 % unit == 0 or k1 == self.in_features), (k0, k1, unit)
        gs = self.group_size
        hb = self.hadamard_block
        assert not hb or (k0 % hb == 0 and (k1 - k0) % hb == 0), "a column shard must not cut a rotation block"
        return FP4ExpertBank(self.qtile[:, :, k0 // 64: (k1 + 63) // 64].contiguous(),
                             self.stile[:, :, k0 // gs: (k1 + gs - 1) // gs].contiguous(), self.out_features, k1 - k0, gs, hb)

    def to(self, device) -> "FP4ExpertBank":
        b = FP4ExpertBank(self.qtile.to(device), self.stile.to(device), self.out_features, self.in_features, self.group_size,
                          self.hadamard_block)
        b.names = self.names
        return b

    def expert(self, e: int) -> FP4Weight:
        return FP4Weight(self.qtile[e], self.stile[e], self.out_features, self.in_features, self.group_size, self.hadamard_block)

    def dequantize(self, dtype=torch.float32, cache: bool = False) -> torch.Tensor:
        if self._deq is not None and self._deq.dtype == dtype:
            return self._deq
        w = torch.stack([self.expert(e).dequantize(dtype) for e in range(self.num_experts)])
        if cache:
            self._deq = w
        return w

    def nbytes(self) -> int:
        return self.qtile.numel() * 4 + self.stile.numel() * 2
