"""Quantize the matrices of a checkpoint in this package's formats, measure, report and draw."""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, List, Optional, Sequence

import torch

from .error_analysis import ErrorAnalyzer, ErrorMetrics
from . import plots

FORMAT_BITS = {"fp4": 4, "int4": 4, "nf4": 4, "int8": 8, "fp8": 8, "int3": 3, "int2": 2, "nf3": 3, "nf2": 2}


def _safe(name: str) -> str:
    return name.replace("/", "_").replace(".", "_")


class WeightVisualizer:
    def __init__(self, weights: Dict[str, torch.Tensor], group_size: int = 128):
        self.weights = {k: v for k, v in weights.items() if torch.is_tensor(v) and v.dim() == 2 and v.is_floating_point()}
        self.group_size = group_size
        self.analyzer = ErrorAnalyzer()
        self._cache: Dict = {}

    @classmethod
    def from_safetensors(cls, path: str, group_size: int = 128, max_tensors: Optional[int] = None, name_filter: Optional[str] = None) -> "WeightVisualizer":
        """``path``: a ``.safetensors`` file or a directory of them; only float matrices are kept (``name_filter``: substring)."""
        from ..formats.safetensors_io import SafetensorsFile
        files = sorted(os.path.join(path, f) for f in os.listdir(path) if f.endswith(".safetensors")) if os.path.isdir(path) else [path]
        out: Dict[str, torch.Tensor] = {}
        for fp in files:
            with SafetensorsFile(fp) as sf:
                for k in sf.keys():
                    if len(sf.shape(k)) == 2 and sf.dtype_str(k) in ("F32", "F16", "BF16") and (name_filter is None or name_filter in k):
                        out[k] = sf.get_tensor(k)
                        if max_tensors is not None and len(out) >= max_tensors:
                            return cls(out, group_size)
        return cls(out, group_size)

    def layer_names(self) -> List[str]:
        return list(self.weights)

    def _group(self, w: torch.Tensor) -> int:
        gs = self.group_size
        while w.shape[1] % gs:
            gs //= 2
        return max(gs, 1)

    def quantize(self, layer_name: str, fmt: str) -> torch.Tensor:
        """The de-quantized round-to-nearest ``fmt`` version of a matrix."""
        key = (layer_name, fmt)
        if key not in self._cache:
            from ..quant import rtn
            w = self.weights[layer_name].float()
            self._cache = {key: rtn.dequantize(rtn.quantize(w, fmt, self._group(w))).float()}     # keep one: matrices are large
        return self._cache[key]

    def bits_per_weight(self, layer_name: str, fmt: str) -> float:
        return FORMAT_BITS[fmt] + 16.0 / self._group(self.weights[layer_name])

    def compare_quantization(self, layer_name: str, fmt: str = "fp4") -> ErrorMetrics:
        if layer_name not in self.weights:
            raise KeyError(f"no matrix named {layer_name!r}")
        if fmt not in FORMAT_BITS:
            raise ValueError(f"unknown format {fmt!r}; options: {sorted(FORMAT_BITS)}")
        m = ErrorMetrics.from_tensors(self.weights[layer_name].float(), self.quantize(layer_name, fmt), self.bits_per_weight(layer_name, fmt))
        self.analyzer.add_layer_metrics(layer_name, fmt, m)
        return m

    def compare_formats(self, layer_name: str, formats: Sequence[str] = ("fp4", "int4", "nf4", "int8")) -> Dict[str, ErrorMetrics]:
        return {f: self.compare_quantization(layer_name, f) for f in formats}

    def plot_error_heatmap(self, layer_name: str, fmt: str = "fp4", path: Optional[str] = None):
        return plots.plot_error_heatmap(self.weights[layer_name].float(), self.quantize(layer_name, fmt), path, title=f"{layer_name} [{fmt}]")

    def plot_weight_comparison(self, layer_name: str, fmt: str = "fp4", path: Optional[str] = None):
        return plots.plot_weight_comparison(self.weights[layer_name].float(), self.quantize(layer_name, fmt), path, title=fmt)

    def plot_error_distribution(self, layer_name: str, formats: Sequence[str] = ("fp4",), path: Optional[str] = None):
        w = self.weights[layer_name].float()
        return plots.plot_error_distribution({f: self.quantize(layer_name, f) - w for f in formats}, path, title=layer_name[-40:])

    def generate_error_report(self, output_dir: str, formats: Sequence[str] = ("fp4",), layers: Optional[Iterable[str]] = None, plots_for_worst: int = 3
                              ) -> Dict:
        """Measures every (layer, format), writes ``error_report.json`` (per layer and per format), ``layer_errors_<fmt>.png`` and, for the
        ``plots_for_worst`` layers with the largest RMSE in the first format, a heat map and a comparison picture."""
        os.makedirs(output_dir, exist_ok=True)
        for name in (list(layers) if layers is not None else self.layer_names()):
            for f in formats:
                self.compare_quantization(name, f)
        report = self.analyzer.to_dict()
        report["best_format_per_layer"] = {k: {"format": f, "rmse": v} for k, (f, v) in self.analyzer.get_best_format_per_layer("rmse").items()}
        report["problematic_layers"] = {f: self.analyzer.identify_problematic_layers(f, top_k=10) for f in formats}
        with open(os.path.join(output_dir, "error_report.json"), "w") as fh:
            json.dump(report, fh, indent=1)
        for f in formats:
            errs = {l: fm[f].rmse for l, fm in self.analyzer.layer_metrics.items() if f in fm}
            plots.plot_layer_errors(errs, os.path.join(output_dir, f"layer_errors_{f}.png"), title=f)
        for name, _ in self.analyzer.identify_problematic_layers(formats[0], top_k=plots_for_worst):
            self.plot_error_heatmap(name, formats[0], os.path.join(output_dir, f"heatmap_{_safe(name)}_{formats[0]}.png"))
            self.plot_weight_comparison(name, formats[0], os.path.join(output_dir, f"compare_{_safe(name)}_{formats[0]}.png"))
        return report
