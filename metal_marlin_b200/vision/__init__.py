"""Vision front end for vision-language models: GPU image preprocessing, multimodal projectors, encoder cache.

Parity: reference ``metal_marlin/vision/*`` — preprocessing on the GPU (resize / normalise / patch extraction; Metal
kernels there, ``csrc/vision.cu`` here), projectors (LLaVA two-layer MLP, Qwen2-VL patch merger, InternVL pixel-shuffle
MLP, perceiver resampler) and the encoder quantization config; ``VisionEncoderCache`` from
``metal_marlin/paged/allocator.py:878`` (content-hash -> encoded image tokens, LRU).
"""
from __future__ import annotations

import hashlib
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import ops

CLIP_MEAN, CLIP_STD = (0.48145466, 0.4578275, 0.40821073), (0.26862954, 0.26130258, 0.27577711)
IMAGENET_MEAN, IMAGENET_STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)


@dataclass
class PreprocessConfig:
    image_size: int = 336
    patch_size: int = 14
    mean: Tuple[float, float, float] = CLIP_MEAN
    std: Tuple[float, float, float] = CLIP_STD
    as_patches: bool = True
    resample: str = "bilinear"          # "bilinear" | "bicubic" | "nearest"
    crop: str = "none"                  # "center": largest centred square (CLIP-style resize + centre crop in one pass)
    merge_size: int = 1                 # > 1: patches ordered by merge x merge groups (Qwen2-VL spatial merge)


def center_crop_box(height: int, width: int, aspect: float = 1.0) -> Tuple[int, int, int, int]:
    """``(y, x, h, w)`` of the largest centred rectangle with the given width / height aspect ratio."""
    if width / height > aspect:
        h, w = height, max(1, int(round(height * aspect)))
    else:
        h, w = max(1, int(round(width / aspect))), width
    return (height - h) // 2, (width - w) // 2, h, w


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280) -> Tuple[int, int]:
    """Dynamic resolution of Qwen2-VL style encoders: the size closest to the image whose sides are multiples of ``factor``
    (patch x merge) and whose area lies in ``[min_pixels, max_pixels]``, keeping the aspect ratio."""
    import math
    if max(height, width) / min(height, width) > 200:
        raise ValueError("aspect ratio above 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def preprocess_dynamic(image: torch.Tensor, patch: int = 14, merge: int = 2, resample: str = "bicubic", mean=CLIP_MEAN, std=CLIP_STD,
                       min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280):
    """One image of any size -> ``(patches [n, 3 * patch^2] in merge-group order, (grid_h, grid_w))`` at its dynamic
    resolution (one kernel launch)."""
    H, W = image.shape[-3], image.shape[-2]
    oh, ow = smart_resize(H, W, patch * merge, min_pixels, max_pixels)
    out = ops.vision_preprocess_ex(image.unsqueeze(0) if image.dim() == 3 else image, oh, ow, patch=patch, merge=merge, resample=resample,
                                   mean=mean, std=std)
    return out[0], (oh // patch, ow // patch)


def channel_statistics(images: torch.Tensor) -> torch.Tensor:
    """fp32 ``[B, 3, 2]``: per-image, per-channel mean and standard deviation of ``pixel / 255``."""
    return ops.channel_stats(images if images.dim() == 4 else images.unsqueeze(0))


class ImagePreprocessor:
    """uint8 HWC images -> normalised bf16 pixels or flattened patches, one kernel launch per batch."""

    def __init__(self, cfg: Optional[PreprocessConfig] = None, device=None):
        self.cfg = cfg or PreprocessConfig()
        self.device = device

    def __call__(self, images) -> torch.Tensor:
        """``images``: uint8 tensor ``[B, H, W, 3]`` or a list of ``[H, W, 3]`` tensors of one size."""
        if isinstance(images, (list, tuple)):
            images = torch.stack([torch.as_tensor(i) for i in images])
        if images.dim() == 3:
            images = images.unsqueeze(0)
        if self.device is not None:
            images = images.to(self.device)
        c = self.cfg
        if c.resample == "bilinear" and c.crop == "none" and c.merge_size == 1:
            return ops.vision_preprocess(images.contiguous(), c.image_size, c.image_size, patch=c.patch_size if c.as_patches else 0, mean=c.mean, std=c.std)
        crop = center_crop_box(images.shape[1], images.shape[2]) if c.crop == "center" else None
        return ops.vision_preprocess_ex(images.contiguous(), c.image_size, c.image_size, crop=crop, patch=c.patch_size if c.as_patches else 0,
                                        merge=c.merge_size, resample=c.resample, mean=c.mean, std=c.std)

    def num_patches(self) -> int:
        return (self.cfg.image_size // self.cfg.patch_size) ** 2


def dynamic_tiles(height: int, width: int, tile: int = 448, max_tiles: int = 12) -> Tuple[int, int]:
    """InternVL-style dynamic resolution: the (rows, cols) tile grid whose aspect ratio is closest to the image's."""
    best, best_diff = (1, 1), float("inf")
    ar = width / height
    for n in range(1, max_tiles + 1):
        for r in range(1, n + 1):
            if n % r:
                continue
            c = n // r
            diff = abs(ar - c / r)
            if diff < best_diff or (diff == best_diff and r * c > best[0] * best[1] and height * width > 0.5 * tile * tile * r * c):
                best, best_diff = (r, c), diff
    return best


# ------------------------------------------------------------------------------------------ projectors
class LlavaProjector:
    """Two-layer MLP with GELU from the vision width to the language width."""

    def __init__(self, w1, b1, w2, b2):
        self.w1, self.b1, self.w2, self.b2 = w1, b1, w2, b2

    def __call__(self, feats: torch.Tensor) -> torch.Tensor:
        h = F.gelu(F.linear(feats.to(self.w1.dtype), self.w1, self.b1))
        return F.linear(h, self.w2, self.b2)


class PatchMergerProjector:
    """Qwen2-VL merger: LayerNorm, concatenate each ``merge x merge`` neighbourhood of patches, two-layer MLP."""

    def __init__(self, ln_w, ln_b, w1, b1, w2, b2, merge: int = 2):
        self.ln_w, self.ln_b, self.w1, self.b1, self.w2, self.b2, self.merge = ln_w, ln_b, w1, b1, w2, b2, merge

    def __call__(self, feats: torch.Tensor, grid_hw: Tuple[int, int]) -> torch.Tensor:
        B, N, C = feats.shape
        h, w = grid_hw
        m = self.merge
        x = ops.layernorm(feats.to(self.w1.dtype), self.ln_w, self.ln_b)
        x = x.view(B, h // m, m, w // m, m, C).permute(0, 1, 3, 2, 4, 5).reshape(B, (h // m) * (w // m), m * m * C)
        return F.linear(F.gelu(F.linear(x, self.w1, self.b1)), self.w2, self.b2)


class PixelShuffleProjector:
    """InternVL: pixel-shuffle down-sampling by ``scale`` (fewer, wider tokens), LayerNorm, two-layer MLP."""

    def __init__(self, ln_w, ln_b, w1, b1, w2, b2, scale: float = 0.5):
        self.ln_w, self.ln_b, self.w1, self.b1, self.w2, self.b2, self.scale = ln_w, ln_b, w1, b1, w2, b2, scale

    def __call__(self, feats: torch.Tensor) -> torch.Tensor:
        B, N, C = feats.shape
        s = int(N ** 0.5)
        r = int(round(1 / self.scale))
        x = feats.view(B, s, s, C).view(B, s, s // r, C * r).permute(0, 2, 1, 3).reshape(B, s // r, s // r, C * r * r)
        x = x.permute(0, 2, 1, 3).reshape(B, (s // r) ** 2, C * r * r).to(self.w1.dtype)
        x = ops.layernorm(x, self.ln_w, self.ln_b)
        return F.linear(F.gelu(F.linear(x, self.w1, self.b1)), self.w2, self.b2)


class PerceiverResampler:
    """A fixed set of learned latent queries cross-attends to the image features (one layer)."""

    def __init__(self, latents, wq, wk, wv, wo, n_heads: int = 8):
        self.latents, self.wq, self.wk, self.wv, self.wo, self.n_heads = latents, wq, wk, wv, wo, n_heads

    def __call__(self, feats: torch.Tensor) -> torch.Tensor:
        B = feats.shape[0]
        L, D = self.latents.shape
        H = self.n_heads
        q = F.linear(self.latents, self.wq).view(1, L, H, D // H).transpose(1, 2).expand(B, -1, -1, -1)
        k = F.linear(feats.to(self.wk.dtype), self.wk).view(B, -1, H, D // H).transpose(1, 2)
        v = F.linear(feats.to(self.wv.dtype), self.wv).view(B, -1, H, D // H).transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, L, D)
        return F.linear(o, self.wo)


def merge_image_tokens(text_embeds: torch.Tensor, image_embeds: torch.Tensor, input_ids: torch.Tensor, image_token_id: int) -> torch.Tensor:
    """Scatter projected image tokens into the positions of ``image_token_id`` placeholders (row-major order)."""
    mask = input_ids == image_token_id
    n = int(mask.sum())
    flat = image_embeds.reshape(-1, image_embeds.shape[-1])
    if n != flat.shape[0]:
        raise ValueError(f"{n} image placeholders but {flat.shape[0]} image tokens")
    out = text_embeds.clone()
    out[mask] = flat.to(out.dtype)
    return out


@dataclass
class VisionQuantConfig:
    """Which parts of the vision tower are quantized: attention / MLP projections to ``fmt``; patch embedding, position
    embeddings, norms and the projector stay in 16 bit (they are small and sensitive)."""
    fmt: str = "int8"
    group_size: int = 128
    skip: Tuple[str, ...] = ("patch_embed", "pos_embed", "norm", "projector", "merger", "cls_token")

    def should_quantize(self, name: str, shape: Sequence[int]) -> bool:
        return len(shape) == 2 and min(shape) >= 64 and not any(s in name for s in self.skip)


class VisionEncoderCache:
    """Content-addressed LRU of encoded images so a repeated image is not re-encoded."""

    def __init__(self, max_entries: int = 64):
        self.max_entries = max_entries
        self._d: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        self.hits = self.misses = 0

    @staticmethod
    def key(image: torch.Tensor) -> str:
        return hashlib.sha256(image.detach().cpu().contiguous().numpy().tobytes()).hexdigest()

    def get_or_encode(self, image: torch.Tensor, encode) -> torch.Tensor:
        k = self.key(image)
        if k in self._d:
            self.hits += 1
            self._d.move_to_end(k)
            return self._d[k]
        self.misses += 1
        v = encode(image)
        self._d[k] = v
        while len(self._d) > self.max_entries:
            self._d.popitem(last=False)
        return v


__all__ = ["PreprocessConfig", "ImagePreprocessor", "dynamic_tiles", "LlavaProjector", "PatchMergerProjector", "PixelShuffleProjector",
           "PerceiverResampler", "merge_image_tokens", "VisionQuantConfig", "VisionEncoderCache", "CLIP_MEAN", "CLIP_STD",
           "LLaVAProjector", "Qwen2VLProjector", "InternVLProjector", "VisionProjector", "VisionProjectorConfig", "detect_projector_type", "VisionMetal",
           "VisionDevice", "preprocess_for_vit", "VisionCalibrationConfig", "VisionCalibrationDataset", "build_vision_calibration_dataset",
           "collect_vision_calibration_stats", "analyze_vision_encoder_sensitivity", "build_vision_precision_map", "build_vlm_precision_map",
           "pack_vlm_mixed_format", "VisionLayerType", "VisionLayerSensitivity", "SensitivityReport", "classify_vision_layer"]


# ------------------------------------------------------------------------------------------------ the reference's names
LLaVAProjector = LlavaProjector
Qwen2VLProjector = PatchMergerProjector
InternVLProjector = PixelShuffleProjector

_LAZY = {
    "VisionProjector": ("..compat_api", "VisionProjector"), "VisionProjectorConfig": ("..compat_api", "VisionProjectorConfig"),
    "detect_projector_type": ("..compat_api", "detect_projector_type"),
    "VisionMetal": (".device_ops", "VisionMetal"), "VisionDevice": (".device_ops", "VisionDevice"), "preprocess_for_vit": (".device_ops", "preprocess_for_vit"),
    **{n: (".calibration", n) for n in (
        "VisionCalibrationConfig", "VisionCalibrationDataset", "build_vision_calibration_dataset", "collect_vision_calibration_stats",
        "analyze_vision_encoder_sensitivity", "build_vision_precision_map", "build_vlm_precision_map", "pack_vlm_mixed_format", "VisionLayerType",
        "VisionLayerSensitivity", "SensitivityReport", "classify_vision_layer")},
}


def __getattr__(name: str):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod, __package__), attr)
    raise AttributeError(name)
