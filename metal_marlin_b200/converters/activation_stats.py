"""Activation statistics for scale calibration of ``torch.nn`` models: text calibration sets, a hook-based collector
(min / max / absmax and clipping percentiles of every Linear's input) and the scale rule that turns them into FP4 / INT4
ranges.

The percentile estimate is streaming: one fixed-size histogram per layer over a symmetric range that doubles whenever a
batch exceeds it (neighbouring bins are merged pairwise, so counts stay exact and memory stays constant); ``method="exact"``
keeps the values and uses ``torch.quantile``-style order statistics instead.

Parity: reference ``converters/calibration.py`` (``CalibrationDataset`` :69 with ``bartowski_v3`` / ``from_file`` / ``from_texts`` /
``tokenize``; ``CalibrationStats`` :227; ``CalibrationCollector`` :254 with ``get_stats`` / ``remove_hooks`` / ``reset`` / ``num_layers``;
``compute_scales`` :440).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

_CALIBRATION_DIRS = ("MMB200_CALIBRATION_DIR",)


@dataclass
class CalibrationDataset:
    """Calibration texts.  ``bartowski_v3`` reads ``calibration_datav3.txt`` from a local directory (``cache_dir``, else the
    directory named by ``MMB200_CALIBRATION_DIR``, else ``~/.cache/metal_marlin_b200/calibration``); nothing is downloaded."""
    samples: List[str] = field(default_factory=list)
    name: str = "custom"
    source: str = "custom"

    def __len__(self) -> int:
        return len(self.samples)

    def __iter__(self):
        return iter(self.samples)

    def __getitem__(self, i):
        return self.samples[i]

    @classmethod
    def from_texts(cls, texts: Sequence[str], name: str = "custom") -> "CalibrationDataset":
        return cls(list(texts), name, "custom")

    @classmethod
    def from_file(cls, path: str, max_samples: Optional[int] = None, min_chars: int = 1, name: Optional[str] = None,
                  source: Optional[str] = None) -> "CalibrationDataset":
        """Samples are the blank-line-separated paragraphs of the file (every non-empty line when it has no blank lines)."""
        with open(path, encoding="utf-8", errors="replace") as f:
            text = f.read()
        parts = [p.strip() for p in text.split("\n\n")]
        if len([p for p in parts if p]) <= 1:
            parts = [ln.strip() for ln in text.splitlines()]
        parts = [p for p in parts if len(p) >= min_chars]
        if max_samples is not None:
            parts = parts[:max_samples]
        return cls(parts, name or os.path.splitext(os.path.basename(path))[0], source or str(path))

    @classmethod
    def bartowski_v3(cls, max_samples: Optional[int] = None, cache_dir: Optional[str] = None) -> "CalibrationDataset":
        dirs = [cache_dir] if cache_dir else []
        dirs += [os.environ[e] for e in _CALIBRATION_DIRS if os.environ.get(e)]
        dirs.append(os.path.join(os.path.expanduser("~"), ".cache", "metal_marlin_b200", "calibration"))
        for d in dirs:
            p = os.path.join(d, "calibration_datav3.txt")
            if os.path.isfile(p):
                return cls.from_file(p, max_samples, min_chars=16, name="bartowski-v3")
        raise FileNotFoundError("calibration_datav3.txt not found in " + ", ".join(dirs) + " (this build has no network access; place the file there)")

    def tokenize(self, tokenizer, max_length: int = 2048, return_tensors: str = "pt") -> list:
        """One encoding per sample.  A Hugging Face tokenizer is called as such; an object with only ``encode`` gives
        ``{"input_ids", "attention_mask"}`` padded with zeros to ``max_length``."""
        out = []
        for text in self.samples:
            if callable(tokenizer):
                out.append(tokenizer(text, max_length=max_length, truncation=True, padding="max_length", return_tensors=return_tensors))
                continue
            ids = list(tokenizer.encode(text))[:max_length]
            mask = [1] * len(ids) + [0] * (max_length - len(ids))
            ids = ids + [0] * (max_length - len(ids))
            if return_tensors == "pt":
                out.append({"input_ids": torch.tensor([ids]), "attention_mask": torch.tensor([mask])})
            else:
                import numpy as np
                out.append({"input_ids": np.asarray([ids]), "attention_mask": np.asarray([mask])})
        return out


@dataclass
class CalibrationStats:
    min_val: torch.Tensor
    max_val: torch.Tensor
    absmax: torch.Tensor
    percentile_low: Optional[torch.Tensor] = None
    percentile_high: Optional[torch.Tensor] = None
    num_batches: int = 0


class _RangeHistogram:
    """Counts over ``[-limit, limit)`` in ``bins`` equal bins; ``limit`` doubles (bins merged pairwise around the centre) until
    a batch fits."""

    def __init__(self, bins: int):
        assert bins % 4 == 0
        self.bins = bins
        self.limit = 0.0
        self.counts = torch.zeros(bins, dtype=torch.float64)

    def _double(self) -> None:
        merged = self.counts.view(-1, 2).sum(1)                 # bins / 2 bins covering the old range
        q = self.bins // 4
        self.counts = torch.cat([torch.zeros(q, dtype=torch.float64), merged, torch.zeros(q, dtype=torch.float64)])
        self.limit *= 2

    def add(self, x: torch.Tensor) -> None:
        x = x.detach().reshape(-1).to(torch.float32).cpu()
        if x.numel() == 0:
            return
        top = float(x.abs().max())
        if self.limit == 0.0:
            self.limit = max(top * 1.0001, 1e-12)
        while top >= self.limit:
            self._double()
        idx = ((x + self.limit) * (self.bins / (2 * self.limit))).long().clamp_(0, self.bins - 1)
        self.counts += torch.bincount(idx, minlength=self.bins).to(torch.float64)

    def percentile(self, p: float) -> float:
        total = float(self.counts.sum())
        if total == 0:
            return 0.0
        target = total * p / 100.0
        cum = torch.cumsum(self.counts, 0)
        i = int(torch.searchsorted(cum, torch.tensor(target, dtype=torch.float64)).clamp(max=self.bins - 1))
        before = float(cum[i - 1]) if i > 0 else 0.0
        inside = float(self.counts[i])
        frac = (target - before) / inside if inside > 0 else 0.0
        width = 2 * self.limit / self.bins
        return -self.limit + (i + min(max(frac, 0.0), 1.0)) * width


class CalibrationCollector:
    """Forward pre-hooks on the ``nn.Linear`` modules of ``model`` (all of them, or those whose qualified name starts with one
    of ``layers_to_calibrate``); every forward pass updates the statistics of each hooked layer's input."""

    def __init__(self, model: nn.Module, layers_to_calibrate: Optional[Sequence[str]] = None, percentile_low: float = 0.01,
                 percentile_high: float = 99.99, method: str = "histogram", num_bins: int = 2048):
        if method not in ("histogram", "exact"):
            raise ValueError(f"method must be 'histogram' or 'exact', got {method!r}")
        self.percentile_low, self.percentile_high, self.method, self.num_bins = percentile_low, percentile_high, method, num_bins
        self.stats: Dict[str, CalibrationStats] = {}
        self._hist: Dict[str, _RangeHistogram] = {}
        self._values: Dict[str, List[torch.Tensor]] = {}
        self._handles = []
        for name, mod in model.named_modules():
            if isinstance(mod, nn.Linear) and (layers_to_calibrate is None or any(name.startswith(p) for p in layers_to_calibrate)):
                self._handles.append(mod.register_forward_pre_hook(self._make_hook(name)))
        self._hooked = len(self._handles)

    def _make_hook(self, name: str):
        def hook(_mod, args):
            x = args[0].detach()
            lo, hi = x.min().float().cpu(), x.max().float().cpu()
            s = self.stats.get(name)
            if s is None:
                self.stats[name] = CalibrationStats(lo, hi, torch.maximum(lo.abs(), hi.abs()), num_batches=1)
            else:
                s.min_val, s.max_val = torch.minimum(s.min_val, lo), torch.maximum(s.max_val, hi)
                s.absmax = torch.maximum(s.absmax, torch.maximum(lo.abs(), hi.abs()))
                s.num_batches += 1
            if self.method == "histogram":
                self._hist.setdefault(name, _RangeHistogram(self.num_bins)).add(x)
            else:
                self._values.setdefault(name, []).append(x.reshape(-1).float().cpu())
        return hook

    def get_stats(self) -> Dict[str, CalibrationStats]:
        for name, s in self.stats.items():
            if self.method == "histogram":
                h = self._hist[name]
                lo, hi = h.percentile(self.percentile_low), h.percentile(self.percentile_high)
            else:
                v = torch.cat(self._values[name]).sort().values
                pick = lambda p: float(v[min(v.numel() - 1, max(0, int(round(p / 100.0 * (v.numel() - 1)))))])   # noqa: E731
                lo, hi = pick(self.percentile_low), pick(self.percentile_high)
            s.percentile_low = torch.tensor(max(lo, float(s.min_val)))
            s.percentile_high = torch.tensor(min(hi, float(s.max_val)))
        return self.stats

    def remove_hooks(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []

    def reset(self) -> None:
        self.stats.clear()
        self._hist.clear()
        self._values.clear()

    @property
    def num_layers(self) -> int:
        return self._hooked

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.remove_hooks()
        return False


def compute_scales(stats: Dict[str, CalibrationStats], quant_type: str = "fp4", use_percentile: bool = True
                   ) -> Dict[str, Tuple[torch.Tensor, Optional[torch.Tensor]]]:
    """``{layer: (scale, zero)}``: ``fp4`` maps the clipped magnitude to the largest E2M1 value (6), ``int4_sym`` to 7, and
    ``int4_asym`` spreads ``[low, high]`` over the 16 unsigned codes with a zero point; ``zero`` is ``None`` for the symmetric kinds."""
    out: Dict[str, Tuple[torch.Tensor, Optional[torch.Tensor]]] = {}
    tiny = torch.tensor(1e-8)
    for name, s in stats.items():
        clipped = use_percentile and s.percentile_low is not None and s.percentile_high is not None
        lo, hi = (s.percentile_low, s.percentile_high) if clipped else (s.min_val, s.max_val)
        mag = torch.maximum(lo.abs(), hi.abs()) if clipped else s.absmax
        if quant_type == "fp4":
            out[name] = (torch.maximum(mag / 6.0, tiny), None)
        elif quant_type == "int4_sym":
            out[name] = (torch.maximum(mag / 7.0, tiny), None)
        elif quant_type == "int4_asym":
            scale = torch.maximum((hi - lo) / 15.0, tiny)
            out[name] = (scale, torch.clamp(torch.round(-lo / scale), 0, 15))
        else:
            raise ValueError(f"quant_type must be 'fp4', 'int4_sym' or 'int4_asym', got {quant_type!r}")
    return out


# ------------------------------------------------------------------------------------------------ activation ranges of a whole model
class CalibrationDatasetLoader:
    """Named loaders (reference ``calibration_utils.py:138``): ``v3`` is the multi-domain text set (local file, see
    ``CalibrationDataset.bartowski_v3``), ``from_file`` any text file."""

    @classmethod
    def v3(cls, max_samples: Optional[int] = None, cache_dir: Optional[str] = None, force_download: bool = False, min_sample_length: int = 100
           ) -> CalibrationDataset:
        if force_download:
            raise RuntimeError("there is no download path in this build: place calibration_datav3.txt in the calibration directory")
        ds = CalibrationDataset.bartowski_v3(None, cache_dir)
        ds.samples = [s for s in ds.samples if len(s) >= min_sample_length][: max_samples]
        return ds

    @classmethod
    def from_file(cls, path: str, max_samples: Optional[int] = None, min_sample_length: int = 1) -> CalibrationDataset:
        return CalibrationDataset.from_file(path, max_samples, min_sample_length)


def compute_activation_ranges(model, calibration, layers: Optional[Sequence[str]] = None, batch_size: int = 1, max_seq_len: int = 2048,
                              tokenizer=None, verbose: bool = False) -> Dict[str, Tuple[float, float]]:
    """``{layer name: (min, max)}`` of the inputs of a model's linear layers over a calibration set.

    ``model``: a ``torch.nn.Module`` (hooks on its ``nn.Linear`` modules; ``calibration`` is then an iterable of input tensors, or a
    ``CalibrationDataset`` with a ``tokenizer``) or an engine model with ``forward_logits`` (statistics per checkpoint tensor name
    through the operator capture hook; ``calibration``: token-id sequences, or texts with a ``tokenizer``).
    Reference ``calibration_utils.py:318``."""
    def token_seqs():
        for item in calibration:
            if isinstance(item, str):
                if tokenizer is None:
                    raise ValueError("text calibration samples need a tokenizer")
                ids = tokenizer.encode(item) if hasattr(tokenizer, "encode") else tokenizer(item)["input_ids"]
                yield [int(t) for t in ids][:max_seq_len]
            else:
                yield item

    ranges: Dict[str, Tuple[float, float]] = {}

    def note(name: str, x: torch.Tensor):
        lo, hi = float(x.min()), float(x.max())
        old = ranges.get(name)
        ranges[name] = (lo, hi) if old is None else (min(old[0], lo), max(old[1], hi))

    if isinstance(model, nn.Module):
        col = CalibrationCollector(model, layers, method="histogram", num_bins=256)
        with torch.no_grad():
            for item in token_seqs():
                t = torch.as_tensor(item)
                if t.dtype in (torch.int32, torch.int64) and t.dim() == 1:
                    t = t[:max_seq_len].unsqueeze(0)
                model(t)
        col.remove_hooks()
        return {k: (float(s.min_val), float(s.max_val)) for k, s in col.stats.items()}
    from .. import ops

    def hook(kind, W, x, ids):
        names = getattr(W, "names", None)
        if kind != "linear" or not names:
            return
        for name, _rows in names:
            if layers is None or any(name.startswith(p) or p in name for p in layers):
                note(name, x)

    ops.set_capture(hook)
    try:
        with torch.no_grad():
            for i, seq in enumerate(token_seqs()):
                model.forward_logits([int(t) for t in torch.as_tensor(seq).reshape(-1)[:max_seq_len]])
                if verbose:
                    print(f"calibration sample {i + 1}: {len(ranges)} layers tracked")
    finally:
        ops.set_capture(None)
    return ranges


def ranges_to_scales(ranges: Dict[str, Tuple[float, float]], quant_type: str = "fp4") -> Dict[str, float]:
    """One scale per layer from its ``(min, max)``: ``absmax / 6`` (``fp4``), ``/ 7`` (``int4_sym``), ``/ 127`` (``int8_sym``), ``(max - min) / 15``
    (``int4_asym``)."""
    div = {"fp4": 6.0, "int4_sym": 7.0, "int8_sym": 127.0}
    out = {}
    for name, (lo, hi) in ranges.items():
        if quant_type in div:
            out[name] = max(abs(lo), abs(hi)) / div[quant_type] or 1e-8
        elif quant_type == "int4_asym":
            out[name] = (hi - lo) / 15.0 or 1e-8
        else:
            raise ValueError(f"quant_type must be one of fp4, int4_sym, int4_asym, int8_sym; got {quant_type!r}")
    return out


def save_ranges(ranges: Dict[str, Tuple[float, float]], path: str) -> None:
    import json
    os.makedirs(os.path.dirname(os.path.abspath(str(path))), exist_ok=True)
    with open(path, "w") as f:
        json.dump({k: [float(a), float(b)] for k, (a, b) in ranges.items()}, f, indent=1)


def load_ranges(path: str) -> Dict[str, Tuple[float, float]]:
    import json
    with open(path) as f:
        return {k: (float(v[0]), float(v[1])) for k, v in json.load(f).items()}
