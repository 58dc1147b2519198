"""Image operations as one object (resize, normalise, crop, patch extraction, the fused ViT preprocessing), under the
reference's ``VisionMetal`` name.

uint8 ``[N, H, W, 3]`` images take the fused CUDA preprocessing kernel (``ops.vision_preprocess_ex``: crop, resample with
half-pixel centres, normalise, CHW or patch layout in one launch, bf16 out).  Float inputs — an intermediate of a pipeline that
was already converted — use the same sampling rule through ``torch.nn.functional.interpolate`` (``align_corners=False``) and
keep their dtype.  Layout: NCHW unless ``nhwc=True``; NumPy arrays are accepted everywhere.

Parity: reference ``vision/vision_metal.py`` (``VisionMetal`` :61 — ``resize_bilinear`` :236, ``resize_bicubic`` :307, ``normalize`` :370,
``resize_and_normalize`` :462, ``extract_patches`` :555, ``preprocess_qwen2vl`` :631, ``uint8_to_float`` :720, ``center_crop`` :784,
``resize_aspect_ratio_preserve`` :1261; ``preprocess_for_vit`` :1344).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple, Union

import numpy as np
import torch
import torch.nn.functional as F

from .. import ops

IMAGENET_MEAN, IMAGENET_STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)
_NO_MEAN, _NO_STD = (0.0, 0.0, 0.0), (1.0, 1.0, 1.0)


class VisionDevice:
    def __init__(self, device: Optional[Union[str, torch.device]] = None):
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")

    # ------------------------------------------------------------------ helpers
    def _t(self, x) -> torch.Tensor:
        t = torch.from_numpy(np.ascontiguousarray(x)) if isinstance(x, np.ndarray) else x
        return t.to(self.device)

    @staticmethod
    def _nchw(t: torch.Tensor, nhwc: bool) -> torch.Tensor:
        return t.permute(0, 3, 1, 2) if nhwc else t

    @staticmethod
    def _back(t: torch.Tensor, nhwc: bool) -> torch.Tensor:
        return t.permute(0, 2, 3, 1).contiguous() if nhwc else t

    def _resize(self, x, size: Tuple[int, int], mode: str, nhwc: bool, mean=_NO_MEAN, std=_NO_STD, crop=None) -> torch.Tensor:
        t = self._t(x)
        if t.dim() == 3:
            t = t.unsqueeze(0)
        if t.dtype == torch.uint8 and nhwc and t.shape[-1] == 3:
            out = ops.vision_preprocess_ex(t.contiguous(), size[0], size[1], crop=crop, resample=mode, mean=mean, std=std)   # bf16 NCHW in [0, 1]
            return self._back(out, nhwc)
        v = self._nchw(t, nhwc)
        v = v.float() / 255.0 if v.dtype == torch.uint8 else v
        if crop is not None:
            y, x0, h, w = crop
            v = v[:, :, y: y + h, x0: x0 + w]
        out = F.interpolate(v.float(), size=tuple(size), mode=mode, align_corners=False).to(v.dtype) if mode != "nearest" else \
            F.interpolate(v.float(), size=tuple(size), mode="nearest").to(v.dtype)
        if mean is not _NO_MEAN or std is not _NO_STD:
            out = self._normalize_nchw(out, mean, std)
        return self._back(out, nhwc)

    @staticmethod
    def _normalize_nchw(v: torch.Tensor, mean, std) -> torch.Tensor:
        m = torch.as_tensor(mean, dtype=torch.float32, device=v.device).view(1, -1, 1, 1)
        s = torch.as_tensor(std, dtype=torch.float32, device=v.device).view(1, -1, 1, 1)
        return ((v.float() - m) / s).to(v.dtype if v.is_floating_point() else torch.float32)

    # ------------------------------------------------------------------ operations
    def resize_bilinear(self, input, target_size: Tuple[int, int], nhwc: bool = False) -> torch.Tensor:
        return self._resize(input, target_size, "bilinear", nhwc)

    def resize_bicubic(self, input, target_size: Tuple[int, int], nhwc: bool = False) -> torch.Tensor:
        return self._resize(input, target_size, "bicubic", nhwc)

    # the reference's tiled / vectorised variants are scheduling choices of one kernel here
    resize_bilinear_tiled = resize_bilinear_tiled_shared = resize_bilinear_4pixel = resize_bilinear
    resize_bicubic_8x8 = resize_bicubic

    def normalize(self, image, mean: Sequence[float], std: Sequence[float], nhwc: bool = False) -> torch.Tensor:
        t = self._t(image)
        v = self._nchw(t, nhwc)
        v = v.float() / 255.0 if v.dtype == torch.uint8 else v
        return self._back(self._normalize_nchw(v, mean, std), nhwc)

    def resize_and_normalize(self, image, size: Tuple[int, int], mean: Sequence[float], std: Sequence[float], nhwc: bool = False) -> torch.Tensor:
        return self._resize(image, size, "bilinear", nhwc, tuple(mean), tuple(std))

    def preprocess_large_image_fused(self, image, size: Tuple[int, int], mean: Sequence[float] = IMAGENET_MEAN, std: Sequence[float] = IMAGENET_STD,
                                     nhwc: bool = False) -> torch.Tensor:
        return self.resize_and_normalize(image, size, mean, std, nhwc)

    def extract_patches(self, image, patch_size: int) -> torch.Tensor:
        """``[N, H, W, C] -> [N, (H / p) (W / p), p p C]`` (row-major patches, pixels of a patch row by row, channels last)."""
        t = self._t(image)
        N, H, W, C = t.shape
        if H % patch_size or W % patch_size:
            raise ValueError(f"image {H}x{W} is not a multiple of the patch size {patch_size}")
        p = patch_size
        return t.reshape(N, H // p, p, W // p, p, C).permute(0, 1, 3, 2, 4, 5).reshape(N, (H // p) * (W // p), p * p * C)

    def qwen2vl_size(self, height: int, width: int, max_pixels: int = 1024 * 1024, patch_size: int = 14) -> Tuple[int, int]:
        """The aspect-preserving target resolution: both sides multiples of ``patch_size``, at most ``max_pixels`` in all."""
        scale = min(1.0, math.sqrt(max_pixels / float(height * width)))
        h = max(patch_size, int(height * scale) // patch_size * patch_size)
        w = max(patch_size, int(width * scale) // patch_size * patch_size)
        while h * w > max_pixels:
            if h >= w:
                h -= patch_size
            else:
                w -= patch_size
        return h, w

    def preprocess_qwen2vl(self, image, max_pixels: int = 1024 * 1024, patch_size: int = 14, nhwc: bool = False) -> torch.Tensor:
        t = self._t(image)
        H, W = (t.shape[1], t.shape[2]) if nhwc else (t.shape[2], t.shape[3])
        return self._resize(t, self.qwen2vl_size(H, W, max_pixels, patch_size), "bilinear", nhwc)

    def uint8_to_float(self, image: torch.Tensor) -> torch.Tensor:
        return self._t(image).to(torch.float32) / 255.0

    def center_crop(self, image, size: Tuple[int, int], nhwc: bool = False) -> torch.Tensor:
        t = self._t(image)
        H, W = (t.shape[1], t.shape[2]) if nhwc else (t.shape[2], t.shape[3])
        h, w = size
        if h > H or w > W:
            raise ValueError(f"crop {h}x{w} is larger than the image {H}x{W}")
        y, x = (H - h) // 2, (W - w) // 2
        return (t[:, y: y + h, x: x + w, :] if nhwc else t[:, :, y: y + h, x: x + w]).contiguous()

    def resize_aspect_ratio_preserve(self, input, target_size: Tuple[int, int], pad_value: float = 0.0, nhwc: bool = False) -> torch.Tensor:
        """Scale to fit inside ``target_size`` keeping the aspect ratio, centred, the border filled with ``pad_value``."""
        t = self._t(input)
        H, W = (t.shape[1], t.shape[2]) if nhwc else (t.shape[2], t.shape[3])
        th, tw = target_size
        s = min(th / H, tw / W)
        h, w = max(1, min(th, int(round(H * s)))), max(1, min(tw, int(round(W * s))))
        inner = self._nchw(self._resize(t, (h, w), "bilinear", nhwc), nhwc)
        out = torch.full((inner.shape[0], inner.shape[1], th, tw), pad_value, dtype=inner.dtype, device=inner.device)
        y, x = (th - h) // 2, (tw - w) // 2
        out[:, :, y: y + h, x: x + w] = inner
        return self._back(out, nhwc)


VisionMetal = VisionDevice


def preprocess_for_vit(images, target_size: Tuple[int, int] = (224, 224), mean: Sequence[float] = IMAGENET_MEAN, std: Sequence[float] = IMAGENET_STD,
                       device=None) -> torch.Tensor:
    """Resize (bilinear) and normalise a batch for a ViT: ``[N, 3, H, W]`` out.  Input: one tensor / array or a list of them
    (each ``[3, H, W]`` float, or ``[H, W, 3]`` uint8 — sizes may differ inside a list)."""
    vd = VisionDevice(device)
    if isinstance(images, (list, tuple)):
        return torch.cat([preprocess_for_vit(i, target_size, mean, std, device) for i in images])
    t = vd._t(images)
    if t.dim() == 3:
        t = t.unsqueeze(0)
    nhwc = t.dtype == torch.uint8 and t.shape[-1] == 3
    out = vd.resize_and_normalize(t, target_size, mean, std, nhwc=nhwc)
    return out.permute(0, 3, 1, 2).contiguous() if nhwc else out
