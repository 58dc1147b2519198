"""``quantize_model``: a Hugging Face checkpoint directory to a quantized one, with a per-layer error report.

Names of other decoder families are brought to the Llama names first (``name_mapping``); without calibration data the
weights are rounded to nearest, with calibration token sequences the calibrated path runs (Hessians from those
sequences, GPTQ error feedback).  The report is measured afterwards from the written files: every quantized matrix is
read back, de-quantized and compared with its source.

Parity: reference ``converters/quantize.py`` (``LayerReport`` :28, ``QuantizationReport`` :42, ``quantize_model`` :83).
"""
from __future__ import annotations

import json
import math
import os
import time
from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional, Sequence, Tuple

import torch

DEFAULT_SKIP = ("embed", "lm_head", "norm", "layernorm", "wte", "wpe")


@dataclass
class LayerReport:
    name: str
    shape: Tuple[int, ...]
    rms_error: float
    max_error: float
    snr_db: float
    num_elements: int
    group_size: int
    quant_type: str


@dataclass
class QuantizationReport:
    layers: List[LayerReport] = field(default_factory=list)
    num_quantized: int = 0
    num_skipped: int = 0
    total_tensors: int = 0
    avg_rms_error: float = 0.0
    avg_snr_db: float = 0.0
    output_size_mb: float = 0.0
    elapsed_seconds: float = 0.0

    def to_dict(self) -> Dict[str, Any]:
        d = {k: getattr(self, k) for k in ("num_quantized", "num_skipped", "total_tensors", "avg_rms_error", "avg_snr_db", "output_size_mb",
                                           "elapsed_seconds")}
        d["layers"] = [{"name": r.name, "shape": list(r.shape), "rms_error": r.rms_error, "max_error": r.max_error, "snr_db": r.snr_db,
                        "quant_type": r.quant_type} for r in self.layers]
        return d


def layer_error(name: str, w: torch.Tensor, wq: torch.Tensor, group_size: int, quant_type: str) -> LayerReport:
    d = (w.float() - wq.float())
    mse = float(d.pow(2).mean())
    power = float(w.float().pow(2).mean())
    snr = 10.0 * math.log10(power / mse) if mse > 0 and power > 0 else float("inf")
    return LayerReport(name, tuple(w.shape), math.sqrt(mse), float(d.abs().max()), snr, w.numel(), group_size, quant_type)


def _mapped_stream(model_path: str, model_type: str, config) -> Iterator[Tuple[str, torch.Tensor]]:
    from ..quant.convert import iter_safetensors_weights
    from .name_mapping import map_weight_names
    for name, t in iter_safetensors_weights(model_path):
        yield from map_weight_names({name: t}, model_type, config=config).items()


def quantize_model(model_path: str, output_path: str, calibration_data: Optional[Sequence] = None, quant_type: str = "fp4",
                   group_size: int = 128, skip_layers: Optional[Sequence[str]] = None, model_type: str = "auto", compute_error: bool = True,
                   verbose: bool = False, device: Optional[str] = None) -> QuantizationReport:
    """``quant_type``: ``fp4`` (sharded MMFP4 checkpoint) — the format every runtime path of this package serves.  ``skip_layers``:
    name fragments kept in 16 bits on top of the embeddings / head / norms.  Returns the report and writes it to
    ``<output_path>/quantization_report.json``."""
    from ..formats import fp4 as fp4fmt
    from ..formats.mmfp4_loader import MMFP4ModelLoader
    from ..quant.convert import convert_model, iter_safetensors_weights, should_quantize_tensor
    from .name_mapping import detect_model_type, load_config
    if quant_type != "fp4":
        raise ValueError(f"quant_type {quant_type!r}: checkpoints are written in fp4 (use quant.rtn / converters.load_and_quantize for in-memory int4 / int8 / nf4)")
    t0 = time.time()
    model_path, output_path = str(model_path), str(output_path)
    extra = tuple(s.lower() for s in (skip_layers or ()) if s.lower() not in DEFAULT_SKIP)
    cfg = load_config(model_path) if os.path.isfile(os.path.join(model_path, "config.json")) else None
    if model_type == "auto":
        model_type = detect_model_type(k for k, _ in iter_safetensors_weights(model_path))

    if calibration_data is None:
        info = convert_model(model_path, output_path, "mmfp4", group_size, device=device or "cpu", verbose=verbose,
                             tensors=_mapped_stream(model_path, model_type, cfg), extra_skip=extra)
    else:
        from ..quant.pipeline import quantize_checkpoint
        if model_type not in ("llama", "mistral", "qwen2", "gemma") or extra:
            raise ValueError("calibrated quantization reads the checkpoint by its Llama names; map it first (converters.load_mapped_safetensors)")
        info = quantize_checkpoint(model_path, output_path, fmt="mmfp4", method="gptq", group_size=group_size, calibration=list(calibration_data),
                                   num_samples=len(calibration_data), device=device)
    rep = QuantizationReport(total_tensors=int(info.get("tensors", 0)), num_quantized=int(info.get("quantized", 0)))
    rep.num_skipped = rep.total_tensors - rep.num_quantized
    if compute_error:
        loader = MMFP4ModelLoader(output_path, prefetch_workers=0)
        for name, t in _mapped_stream(model_path, model_type, cfg):
            base = name[: -len(".weight")] if name.endswith(".weight") else name
            if not should_quantize_tensor(name, t, extra) or not loader.is_quantized(base):
                continue
            packed, scales, _layout = loader.get_quantized_weight(base)
            codes, sc = fp4fmt.unpack_mmfp4(packed, scales, t.shape[1])
            wq = fp4fmt.dequantize_codes(codes, sc)
            hb = loader.get_hadamard_block_size(base)
            if hb:
                from ..quant.hadamard import rotate_weight
                wq = rotate_weight(wq, hb)
            rep.layers.append(layer_error(name, t, wq, loader.get_group_size(base, group_size), quant_type))
        loader.close()
        finite = [r for r in rep.layers if math.isfinite(r.snr_db)]
        rep.avg_rms_error = sum(r.rms_error for r in rep.layers) / max(1, len(rep.layers))
        rep.avg_snr_db = sum(r.snr_db for r in finite) / max(1, len(finite))
    rep.output_size_mb = sum(os.path.getsize(os.path.join(output_path, f)) for f in os.listdir(output_path) if f.endswith(".safetensors")) / 2 ** 20
    rep.elapsed_seconds = time.time() - t0
    with open(os.path.join(output_path, "quantization_report.json"), "w") as f:
        json.dump(rep.to_dict(), f, indent=1)
    if verbose:
        print(f"quantized {rep.num_quantized} of {rep.total_tensors} tensors, mean SNR {rep.avg_snr_db:.1f} dB, {rep.output_size_mb:.1f} MiB")
    return rep
