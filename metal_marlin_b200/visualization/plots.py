"""Plots as images (``uint8 [H, W, 3]`` arrays, written as PNG when a path is given), drawn with NumPy and Pillow."""
from __future__ import annotations

import os
from typing import Dict, Optional, Sequence

import numpy as np
import torch

WHITE, BLACK, GRID = (255, 255, 255), (0, 0, 0), (200, 200, 200)
BLUE, RED, GREEN = (40, 90, 200), (210, 60, 50), (40, 150, 70)


def _arr(x) -> np.ndarray:
    return x.detach().float().cpu().numpy() if isinstance(x, torch.Tensor) else np.asarray(x, dtype=np.float32)


def _save(img: np.ndarray, path: Optional[str]) -> np.ndarray:
    if path is not None:
        from PIL import Image
        os.makedirs(os.path.dirname(os.path.abspath(str(path))), exist_ok=True)
        Image.fromarray(img).save(str(path))
    return img


def diverging(v: np.ndarray, limit: float) -> np.ndarray:
    """Blue (negative) - white (zero) - red (positive) colour map of ``v`` clipped to ``[-limit, limit]``."""
    t = np.clip(v / (limit if limit > 0 else 1.0), -1, 1)[..., None]
    pos = np.array(WHITE) * (1 - np.maximum(t, 0)) + np.array(RED) * np.maximum(t, 0)
    neg = np.array(WHITE) * (1 - np.maximum(-t, 0)) + np.array(BLUE) * np.maximum(-t, 0)
    return np.where(t >= 0, pos, neg).astype(np.uint8)


def _fit(m: np.ndarray, max_side: int) -> np.ndarray:
    """Down-sample a matrix by block means so neither side exceeds ``max_side`` (a picture of a 4096 x 4096 matrix shows tiles)."""
    for ax in (0, 1):
        n = m.shape[ax]
        if n > max_side:
            f = -(-n // max_side)
            pad = (-n) % f
            if pad:
                m = np.concatenate([m, np.take(m, range(n - pad, n), axis=ax)], axis=ax)
            shape = (m.shape[0] // f, f, m.shape[1]) if ax == 0 else (m.shape[0], m.shape[1] // f, f)
            m = m.reshape(shape).mean(1 if ax == 0 else 2)
    return m


def _label(img: np.ndarray, text: str, xy=(4, 2), color=BLACK) -> np.ndarray:
    from PIL import Image, ImageDraw
    im = Image.fromarray(img)
    ImageDraw.Draw(im).text(xy, text, fill=color)
    return np.asarray(im).copy()


def plot_error_heatmap(original, quantized, path: Optional[str] = None, max_side: int = 512, title: str = "") -> np.ndarray:
    """Signed error ``quantized - original`` of a matrix as a diverging colour map (limit: the 99.5th percentile of ``|error|``)."""
    e = _fit(_arr(quantized).reshape(_arr(original).shape[0], -1) - _arr(original).reshape(_arr(original).shape[0], -1), max_side)
    img = diverging(e, float(np.percentile(np.abs(e), 99.5)) or 1.0)
    if title:
        img = _label(np.concatenate([np.full((16, img.shape[1], 3), 255, np.uint8), img]), title)
    return _save(img, path)


def plot_weight_comparison(original, quantized, path: Optional[str] = None, max_side: int = 256, title: str = "") -> np.ndarray:
    """Three panels side by side: original, quantized (one shared colour scale) and their difference (its own scale)."""
    o = _arr(original)
    o = _fit(o.reshape(o.shape[0], -1), max_side)
    q = _fit(_arr(quantized).reshape(_arr(original).shape[0], -1), max_side)
    lim = float(np.percentile(np.abs(o), 99.5)) or 1.0
    d = q - o
    gap = np.full((o.shape[0], 6, 3), 255, np.uint8)
    img = np.concatenate([diverging(o, lim), gap, diverging(q, lim), gap, diverging(d, float(np.percentile(np.abs(d), 99.5)) or 1.0)], 1)
    head = np.full((16, img.shape[1], 3), 255, np.uint8)
    w = o.shape[1] + 6
    head = _label(_label(_label(head, (title + " " if title else "") + "original"), "quantized", (w + 4, 2)), "difference", (2 * w + 4, 2))
    return _save(np.concatenate([head, img]), path)


def _axes(h: int, w: int, margin: int = 30):
    img = np.full((h, w, 3), 255, np.uint8)
    img[h - margin, margin:w - 5] = BLACK
    img[5:h - margin, margin] = BLACK
    return img, margin


def plot_error_distribution(errors, path: Optional[str] = None, bins: int = 101, size=(360, 640), title: str = "", log: bool = True) -> np.ndarray:
    """Histogram of an error tensor (or of several: ``{label: tensor}``, one colour each, drawn over one another), counts on a log
    axis by default; symmetric range from the largest 99.9th percentile."""
    series = errors if isinstance(errors, dict) else {"error": errors}
    flat = {k: _arr(v).reshape(-1) for k, v in series.items()}
    lim = max(float(np.percentile(np.abs(v), 99.9)) for v in flat.values()) or 1.0
    h, w = size
    img, m = _axes(h, w)
    colors = [BLUE, RED, GREEN, (150, 80, 170), (230, 150, 30)]
    plot_w, plot_h = w - m - 10, h - m - 25
    hists = {k: np.histogram(np.clip(v, -lim, lim), bins=bins, range=(-lim, lim))[0].astype(np.float64) for k, v in flat.items()}
    top = max(hh.max() for hh in hists.values()) or 1.0
    for ci, (k, hh) in enumerate(hists.items()):
        y = np.log1p(hh) / np.log1p(top) if log else hh / top
        for b in range(bins):
            x0, x1 = m + 1 + b * plot_w // bins, m + 1 + (b + 1) * plot_w // bins
            bar = int(round(y[b] * plot_h))
            if bar > 0:
                if len(hists) == 1:
                    img[h - m - bar:h - m, x0:max(x1 - 1, x0 + 1)] = colors[ci]
                else:
                    img[h - m - bar:h - m - bar + 2, x0:x1] = colors[ci % len(colors)]
    img = _label(img, f"{title}  range +-{lim:.3g}  {'log' if log else 'linear'} counts")
    for ci, k in enumerate(hists):
        img = _label(img, k, (m + 6 + 90 * ci, 14), colors[ci % len(colors)])
    return _save(img, path)


def plot_layer_errors(layer_errors: Dict[str, float], path: Optional[str] = None, metric: str = "rmse", size=(360, 800), title: str = "",
                      highlight_top: int = 5) -> np.ndarray:
    """Bar per layer (in the order given), the ``highlight_top`` largest in red; the names of those are listed in the corner."""
    names, vals = list(layer_errors), np.asarray(list(layer_errors.values()), dtype=np.float64)
    h, w = size
    img, m = _axes(h, w)
    if len(vals):
        plot_w, plot_h = w - m - 10, h - m - 25
        top = float(vals.max()) or 1.0
        worst = set(np.argsort(-vals)[:highlight_top].tolist())
        for i, v in enumerate(vals):
            x0, x1 = m + 1 + i * plot_w // len(vals), m + 1 + (i + 1) * plot_w // len(vals)
            bar = max(1, int(round(v / top * plot_h)))
            img[h - m - bar:h - m, x0:max(x1 - 1, x0 + 1)] = RED if i in worst else BLUE
        img = _label(img, f"{title}  {metric} per layer ({len(vals)} layers), max {top:.4g}")
        for j, i in enumerate(sorted(worst, key=lambda i: -vals[i])):
            img = _label(img, f"{names[i][-48:]}  {vals[i]:.4g}", (m + 6, 14 + 11 * j), RED)
    return _save(img, path)
