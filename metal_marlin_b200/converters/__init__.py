"""Checkpoint importers / converters: GGUF (de-quantize + re-quantize), PyTorch ``.bin`` / ``.pt`` state dicts, HF
safetensors, GPTQ (AutoGPTQ-style int4), EXL3-style trellis tensors and ONNX graphs (``onnx.py``: own protobuf reader,
graph summary, executor with quantized MatMul / Gemm), plus the mixed-format packer; weight-name mapping of other decoder
families (``name_mapping.py``), activation statistics (``activation_stats.py``), the quantize-with-report driver
(``quantize_report.py``) and the quantized custom operators for ONNX graphs (``custom_ops.py``).

Parity: reference ``metal_marlin/converters/*``, ``gguf_to_marlin.py``, ``hf_exl3_loader.py``,
``quantization/exl3_to_marlin.py``, ``packing/mixed_format.py`` and the ``convert`` command (``cli.py:307-345``).
"""
from __future__ import annotations

import json
import os
import shutil
import tempfile
import time
from typing import Dict, Iterator, Optional, Tuple

import torch

from ..formats.safetensors_io import save_file
from . import gguf
from .gptq_import import dequantize_gptq_int4, import_gptq_state
from .mixed_format import MixedFormatPack


def detect_format(path: str) -> str:
    if os.path.isfile(path):
        ext = os.path.splitext(path)[1].lower()
        if ext == ".gguf":
            return "gguf"
        if ext == ".onnx":
            return "onnx"
        if ext == ".nemo":
            return "nemo"
        if ext in (".bin", ".pt", ".pth"):
            return "pytorch"
        if ext == ".safetensors":
            return "safetensors"
    if os.path.isdir(path):
        files = os.listdir(path)
        if any(f.endswith(".gguf") for f in files):
            return "gguf"
        if any(f.endswith(".safetensors") for f in files):
            return "safetensors"
        if any(f.endswith((".bin", ".pt")) for f in files):
            return "pytorch"
    raise ValueError(f"cannot detect the checkpoint format of {path}")


def _iter_source(src: str, fmt: str) -> Iterator[Tuple[str, torch.Tensor]]:
    if fmt == "gguf":
        p = src if os.path.isfile(src) else os.path.join(src, next(f for f in sorted(os.listdir(src)) if f.endswith(".gguf")))
        with gguf.GGUFReader(p) as r:
            for name in r.tensor_names():
                yield gguf.gguf_name_to_hf(name), r.load_tensor(name)
    elif fmt == "nemo":
        from . import nemo as _nemo
        sd, _ = _nemo.load_nemo(src)
        yield from sd.items()
    elif fmt == "onnx":
        # the linear weights of the graph (as [out, in]) plus every other float initializer under its own name
        from . import onnx as _onnx
        g = _onnx.load_onnx(src)
        lin = _onnx.extract_linear_weights(g)
        for k, arr in g.initializers.items():
            if k in lin:
                yield k + ".weight", lin[k]
            elif arr.dtype.kind == "f":
                yield k, torch.from_numpy(arr.astype("float32"))
    elif fmt == "pytorch":
        files = [src] if os.path.isfile(src) else [os.path.join(src, f) for f in sorted(os.listdir(src)) if f.endswith((".bin", ".pt", ".pth"))]
        for fp in files:
            sd = torch.load(fp, map_location="cpu", weights_only=True)
            sd = sd.get("state_dict", sd) if isinstance(sd, dict) else sd
            for k, v in sd.items():
                if isinstance(v, torch.Tensor):
                    yield k, v
    else:
        from ..quant.convert import iter_safetensors_weights
        yield from iter_safetensors_weights(src if os.path.isdir(src) else os.path.dirname(src))


def convert_checkpoint(src: str, dst: str, from_format: str = "auto", to_format: str = "marlin", quant: str = "fp4",
                       group_size: int = 128, dequant_first: bool = False, device: str = "cpu") -> Dict:
    """``to_format``: ``marlin`` (quantize to ``quant``), ``safetensors`` (float re-export), ``gguf`` (F16 / Q8_0 export)."""
    t0 = time.time()
    fmt = detect_format(src) if from_format in ("auto", "hf") else from_format
    os.makedirs(dst, exist_ok=True)
    if to_format == "gguf":
        tensors = {k: v for k, v in _iter_source(src, fmt)}
        types = {k: (gguf.Q8_0 if (quant == "int8" and v.dim() == 2 and v.shape[-1] % 32 == 0) else gguf.F16) for k, v in tensors.items()}
        gguf.write_gguf(os.path.join(dst, "model.gguf"), tensors, {"general.architecture": "llama", "general.name": os.path.basename(src)}, types)
        return {"tensors": len(tensors), "format": "gguf", "seconds": time.time() - t0}
    # everything else goes through a float safetensors staging directory
    stage = dst if to_format == "safetensors" else tempfile.mkdtemp(prefix="mmb200_convert_")
    try:
        tensors = {k: v.to(torch.bfloat16) if v.is_floating_point() else v for k, v in _iter_source(src, fmt)}
        save_file(tensors, os.path.join(stage, "model.safetensors"), metadata={"format": "pt"})
        src_dir = src if os.path.isdir(src) else os.path.dirname(src)
        for fn in ("config.json", "tokenizer.json", "tokenizer_config.json", "generation_config.json"):
            if os.path.exists(os.path.join(src_dir, fn)) and not os.path.exists(os.path.join(stage, fn)):
                shutil.copy(os.path.join(src_dir, fn), os.path.join(stage, fn))
        if to_format == "safetensors":
            return {"tensors": len(tensors), "format": "safetensors", "seconds": time.time() - t0}
        from ..quant.pipeline import quantize_checkpoint
        stats = quantize_checkpoint(stage, dst, fmt=quant, method="rtn", group_size=group_size, device=device)
        stats["source_format"] = fmt
        stats["dequant_first"] = bool(dequant_first or fmt == "gguf")
        return stats
    finally:
        if stage != dst:
            shutil.rmtree(stage, ignore_errors=True)


# the reference's ``converters`` package names, resolved on first use
_LAZY = {
    ".activation_stats": ["CalibrationCollector", "CalibrationDataset", "CalibrationStats", "compute_scales", "CalibrationDatasetLoader",
                          "compute_activation_ranges", "ranges_to_scales", "save_ranges", "load_ranges"],
    ".quantize_report": ["LayerReport", "QuantizationReport", "quantize_model"],
    ".custom_ops": ["MarlinFlashAttentionOp", "MarlinQuantizedLinearOp", "MarlinQuantizedMatMulOp", "MarlinSession", "create_session",
                    "export_with_marlin_ops"],
    ".name_mapping": ["Rule", "detect_model_type", "estimate_memory", "get_supported_architectures", "load_and_quantize", "load_config",
                      "load_mapped_safetensors", "map_weight_names", "register_architecture"],
    ".nemo": ["convert_nemo_to_pytorch", "load_nemo"],
    ".torch_compat": ["export_for_pytorch", "import_from_pytorch"],
    ".mixed_format": ["MixedFormatHeader", "pack_mixed_format_model", "load_mixed_format_model", "get_layer_precision", "merge_mixed_format_models",
                      "build_mixed_pack"],
    ".onnx": ["ONNXExecutor", "ONNXGraph", "ONNXOp", "load_onnx", "save_onnx"],
}
_WHERE = {n: m for m, names in _LAZY.items() for n in names}


def __getattr__(name: str):
    import importlib
    if name == "load_onnx_model":
        return importlib.import_module(".onnx", __package__).load_onnx
    if name in ("onnx", "nemo", "qmi4", "exl3"):
        return importlib.import_module("." + name, __package__)
    mod = _WHERE.get(name)
    if mod is None:
        raise AttributeError(name)
    return getattr(importlib.import_module(mod, __package__), name)


__all__ = sorted(["convert_checkpoint", "detect_format", "gguf", "onnx", "dequantize_gptq_int4", "import_gptq_state", "MixedFormatPack",
                  "load_onnx_model"] + list(_WHERE))
