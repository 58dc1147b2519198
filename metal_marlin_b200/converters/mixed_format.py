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


# ------------------------------------------------------------------------------------------------ whole-model packing by a precision map
from dataclasses import asdict, dataclass, field      # noqa: E402
from typing import Any, List, Tuple                   # noqa: E402

_FLOAT_FORMATS = ("fp16", "bf16", "float", "keep")
_SUFFIXES = (".scales", ".zeros", ".packed", ".weight")


@dataclass
class MixedFormatHeader:
    """What a reader needs to pick the de-quantization path of every tensor (reference ``packing/mixed_format.py:54``)."""
    layer_formats: Dict[str, str] = field(default_factory=dict)
    layer_group_sizes: Dict[str, int] = field(default_factory=dict)
    total_params: int = 0
    quantized_params: int = 0
    average_bits: float = 16.0
    version: int = 1

    def to_json(self) -> str:
        return json.dumps(asdict(self))

    @classmethod
    def from_json(cls, s: str) -> "MixedFormatHeader":
        return cls(**json.loads(s))

    def _key(self, layer_name: str) -> Optional[str]:
        if layer_name in self.layer_formats:
            return layer_name
        for suf in _SUFFIXES:
            if layer_name.endswith(suf) and layer_name[: -len(suf)] in self.layer_formats:
                return layer_name[: -len(suf)]
        return None

    def get_format(self, layer_name: str) -> Optional[str]:
        k = self._key(layer_name)
        return self.layer_formats[k] if k is not None else None

    def get_group_size(self, layer_name: str) -> Optional[int]:
        k = self._key(layer_name)
        return self.layer_group_sizes.get(k) if k is not None else None

    def summary(self) -> str:
        counts: Dict[str, int] = {}
        for f in self.layer_formats.values():
            counts[f] = counts.get(f, 0) + 1
        parts = ", ".join(f"{n} x {f}" for f, n in sorted(counts.items()))
        return (f"mixed-format model v{self.version}: {len(self.layer_formats)} tensors ({parts}); {self.total_params / 1e6:.2f} M parameters, "
                f"{100.0 * self.quantized_params / max(1, self.total_params):.1f} % quantized, {self.average_bits:.2f} bits per weight")

    @classmethod
    def from_manifest(cls, manifest: Dict[str, Dict]) -> "MixedFormatHeader":
        h = cls()
        bits_total = 0.0
        for name, m in manifest.items():
            n = 1
            for d in m["shape"]:
                n *= int(d)
            h.total_params += n
            if m["format"] == "float":
                h.layer_formats[name] = "bf16"
                bits_total += 16.0 * n
            else:
                h.layer_formats[name] = m["format"]
                h.layer_group_sizes[name] = int(m["group_size"])
                h.quantized_params += n
                bits_total += (m["bits"] + 16.0 / max(1, int(m["group_size"]))) * n
        h.average_bits = bits_total / max(1, h.total_params)
        return h


def _format_name(precision: Any) -> str:
    f = str(getattr(precision, "value", precision) or "bf16").lower()
    return {"fp4_e2m1": "fp4", "fp8_e4m3": "fp8"}.get(f, f)


def build_mixed_pack(weights: Dict[str, Any], precision_map: Dict[str, Tuple[Any, int]]) -> MixedFormatPack:
    """Quantize every tensor to its mapped ``(precision, group size)``; tensors without an entry, non-matrices and 16-bit entries
    are stored in bf16.  A group size that does not divide the input width is halved until it does."""
    import numpy as np
    pack = MixedFormatPack()
    for name, w in weights.items():
        t = w if isinstance(w, torch.Tensor) else torch.as_tensor(np.asarray(w))
        prec, gs = precision_map.get(name, (None, 0))
        fmt = _format_name(prec)
        if fmt in _FLOAT_FORMATS or t.dim() != 2 or t.shape[1] % 8:
            pack.add(name, t.to(torch.bfloat16) if t.is_floating_point() else t, "keep")
            continue
        gs = int(gs) or 128
        while t.shape[1] % gs:
            gs //= 2
        pack.add(name, t, fmt, gs)
    return pack


def pack_mixed_format_model(weights: Dict[str, Any], precision_map: Dict[str, Tuple[Any, int]], output_path: str) -> MixedFormatHeader:
    """One ``.safetensors`` file with every tensor in its own format and the header / manifest in the metadata (reference
    ``packing/mixed_format.py:266``).  Returns the header."""
    pack = build_mixed_pack(weights, precision_map)
    os.makedirs(os.path.dirname(os.path.abspath(str(output_path))), exist_ok=True)
    pack.save(str(output_path))
    return MixedFormatHeader.from_manifest(pack.manifest)


def load_mixed_format_model(model_path: str) -> Tuple[Dict[str, torch.Tensor], MixedFormatHeader]:
    """The stored tensors (packed codes, ``.scales``, ``.zeros``, float tensors — nothing is de-quantized) and the header."""
    if not os.path.isfile(str(model_path)):
        raise FileNotFoundError(str(model_path))
    try:
        pack = MixedFormatPack.load(str(model_path))
    except KeyError:
        raise ValueError(f"{model_path}: no mixed-format manifest in the file metadata")
    return pack.tensors, MixedFormatHeader.from_manifest(pack.manifest)


def get_layer_precision(header: MixedFormatHeader, layer_name: str):
    """``(Precision, group size)`` of a stored tensor (``FP16`` and 0 when the header does not know it)."""
    from ..compat_api import Precision
    f = header.get_format(layer_name)
    if f is None:
        return Precision.FP16, 0
    base = f.split("_")[0]
    return Precision(base), int(header.get_group_size(layer_name) or 0)


def merge_mixed_format_models(model_paths: List[str], output_path: str) -> MixedFormatHeader:
    """Shards packed separately into one file; a tensor present in two shards is an error."""
    merged = MixedFormatPack()
    for p in model_paths:
        part = MixedFormatPack.load(str(p))
        dup = set(part.manifest) & set(merged.manifest)
        if dup:
            raise ValueError(f"{p}: tensors already present in an earlier shard: {sorted(dup)[:3]}")
        merged.tensors.update(part.tensors)
        merged.manifest.update(part.manifest)
    merged.save(str(output_path))
    return MixedFormatHeader.from_manifest(merged.manifest)
