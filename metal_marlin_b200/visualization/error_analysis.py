"""Error metrics of a quantized tensor against its original, and their aggregation over layers and formats."""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

LOWER_IS_BETTER = {"mse", "rmse", "mae", "max_error", "mean_relative_error", "median_relative_error", "outlier_ratio"}


@dataclass
class ErrorMetrics:
    mse: float
    rmse: float
    mae: float
    max_error: float
    mean_relative_error: float
    median_relative_error: float
    psnr: float                          # peak (max |original|) signal to noise, dB
    snr: float                           # signal power to noise power, dB
    cosine_similarity: float
    correlation: float
    bits_per_weight: float
    compression_ratio: float             # against 16-bit storage
    outlier_ratio: float                 # share of weights off by more than 10 % of their magnitude
    quantization_skew: float
    quantization_kurtosis: float         # excess kurtosis of the error

    def to_dict(self) -> Dict[str, float]:
        return asdict(self)

    @classmethod
    def from_tensors(cls, original, quantized, bits_per_weight: float = 4.0) -> "ErrorMetrics":
        o = torch.as_tensor(np.asarray(original) if not isinstance(original, torch.Tensor) else original).double().reshape(-1)
        q = torch.as_tensor(np.asarray(quantized) if not isinstance(quantized, torch.Tensor) else quantized).double().reshape(-1).to(o.device)
        if o.numel() != q.numel():
            raise ValueError(f"shape mismatch: {o.numel()} vs {q.numel()} elements")
        e = q - o
        mse = float(e.pow(2).mean())
        power, peak = float(o.pow(2).mean()), float(o.abs().max())
        db = lambda num: 10.0 * math.log10(num / mse) if mse > 0 and num > 0 else float("inf")    # noqa: E731
        nz = o.abs() > 1e-12
        rel = (e[nz].abs() / o[nz].abs()) if bool(nz.any()) else torch.zeros(1, dtype=torch.float64)
        on, qn = float(o.norm()), float(q.norm())
        cos = float(o.dot(q)) / (on * qn) if on > 0 and qn > 0 else 0.0
        oc, qc = o - o.mean(), q - q.mean()
        den = float(oc.norm()) * float(qc.norm())
        sd = float(e.std(unbiased=False))
        ec = e - e.mean()
        skew = float(ec.pow(3).mean()) / sd ** 3 if sd > 0 else 0.0
        kurt = float(ec.pow(4).mean()) / sd ** 4 - 3.0 if sd > 0 else 0.0
        return cls(mse, math.sqrt(mse), float(e.abs().mean()), float(e.abs().max()), float(rel.mean()), float(rel.median()), db(peak * peak), db(power),
                   cos, float(oc.dot(qc)) / den if den > 0 else 0.0, float(bits_per_weight), 16.0 / float(bits_per_weight) if bits_per_weight else 0.0,
                   float((rel > 0.1).double().mean()), skew, kurt)


class ErrorAnalyzer:
    def __init__(self):
        self.layer_metrics: Dict[str, Dict[str, ErrorMetrics]] = {}

    def add_layer_metrics(self, layer_name: str, format_name: str, metrics: ErrorMetrics) -> None:
        self.layer_metrics.setdefault(layer_name, {})[format_name] = metrics

    def formats(self) -> List[str]:
        return sorted({f for m in self.layer_metrics.values() for f in m})

    def get_layer_comparison(self, layer_name: str) -> Optional[Dict[str, ErrorMetrics]]:
        return self.layer_metrics.get(layer_name)

    def get_format_summary(self, format_name: str) -> Dict[str, float]:
        """Mean / max RMSE, mean SNR, cosine and relative error, and the count, over the layers measured in this format."""
        ms = [m[format_name] for m in self.layer_metrics.values() if format_name in m]
        if not ms:
            return {}
        finite = [m.snr for m in ms if math.isfinite(m.snr)]
        return {"num_layers": float(len(ms)), "mean_rmse": float(np.mean([m.rmse for m in ms])), "max_rmse": float(max(m.rmse for m in ms)),
                "mean_mae": float(np.mean([m.mae for m in ms])), "mean_snr": float(np.mean(finite)) if finite else float("inf"),
                "min_cosine_similarity": float(min(m.cosine_similarity for m in ms)), "mean_relative_error": float(np.mean([m.mean_relative_error for m in ms])),
                "mean_outlier_ratio": float(np.mean([m.outlier_ratio for m in ms])), "bits_per_weight": float(np.mean([m.bits_per_weight for m in ms]))}

    @property
    def format_summaries(self) -> Dict[str, Dict[str, float]]:
        return {f: self.get_format_summary(f) for f in self.formats()}

    def get_best_format_per_layer(self, metric: str = "rmse") -> Dict[str, Tuple[str, float]]:
        out = {}
        for layer, fm in self.layer_metrics.items():
            pick = min if metric in LOWER_IS_BETTER else max
            f = pick(fm, key=lambda k: getattr(fm[k], metric))
            out[layer] = (f, float(getattr(fm[f], metric)))
        return out

    def identify_problematic_layers(self, format_name: str, threshold_rmse: Optional[float] = None, top_k: int = 10) -> List[Tuple[str, float]]:
        rows = [(l, fm[format_name].rmse) for l, fm in self.layer_metrics.items() if format_name in fm
                and (threshold_rmse is None or fm[format_name].rmse > threshold_rmse)]
        return sorted(rows, key=lambda r: -r[1])[:top_k]

    def to_dict(self) -> Dict:
        return {"layers": {l: {f: m.to_dict() for f, m in fm.items()} for l, fm in self.layer_metrics.items()}, "formats": self.format_summaries}
