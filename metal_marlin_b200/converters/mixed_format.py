"""Mixed-format pack: one safetensors file holding tensors in different quantization formats with a manifest.

Parity: reference ``metal_marlin/packing/mixed_format.py``: every entry records its format, bits, group size and
original shape so a loader can build the right layer for each tensor.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch

from ..formats.safetensors_io import SafetensorsFile, save_file
from ..quant import rtn


class MixedFormatPack:
    def __init__(self):
        self.tensors: Dict[str, torch.Tensor] = {}
        self.manifest: Dict[str, Dict] = {}

    def add(self, name: str, w: torch.Tensor, fmt: str = "fp4", group_size: int = 128):
        if fmt == "keep":
            self.tensors[name] = w
            self.manifest[name] = {"format": "float", "shape": list(w.shape)}
            return
        q = rtn.quantize(w.to(torch.float32), fmt, group_size)
        self.tensors[name] = rtn.pack_bits(q.codes, q.bits)
        self.tensors[name + ".scales"] = q.scales
        if q.zeros is not None:
            self.tensors[name + ".zeros"] = q.zeros
        self.manifest[name] = {"format": q.fmt, "bits": q.bits, "group_size": q.group_size, "shape": list(w.shape)}

    def save(self, path: str):
        save_file(self.tensors, path, metadata={"mixed_format_manifest": json.dumps(self.manifest)})

    @classmethod
    def load(cls, path: str) -> "MixedFormatPack":
        p = cls()
        with SafetensorsFile(path) as sf:
            p.manifest = json.loads(sf.metadata["mixed_format_manifest"])
            for k in sf.keys():
                p.tensors[k] = sf.get_tensor(k)
        return p

    def dequantize(self, name: str, dtype=torch.float32) -> torch.Tensor:
        m = self.manifest[name]
        if m["format"] == "float":
            return self.tensors[name].to(dtype)
        out_f, in_f = m["shape"]
        codes = rtn.unpack_bits(self.tensors[name], m["bits"], in_f).view(out_f, in_f)
        q = rtn.QuantizedTensor(codes, self.tensors[name + ".scales"], self.tensors.get(name + ".zeros"), m["format"], m["group_size"], m["bits"])
        return q.dequantize(dtype)
