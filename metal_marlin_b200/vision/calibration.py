"""Calibration and precision planning for the vision tower of a vision-language model: image calibration sets, activation /
Hessian collection on the tower's Linear layers, per-layer sensitivity from simulated quantization error, and the
precision maps (vision tower in 8 / 16 bits, language model in 4) handed to the mixed-format packer.

Parity: reference ``vision/encoder_quant.py`` (``VisionCalibrationConfig`` :75, ``build_vision_calibration_dataset`` :89,
``collect_vision_calibration_stats`` :163, ``analyze_vision_encoder_sensitivity`` :231, ``build_vision_precision_map`` :249,
``build_vlm_precision_map`` :288, ``pack_vlm_mixed_format`` :326), ``vision/image_calibration.py`` (``VisionCalibrationDataset`` :170) and
``vision/layer_sensitivity.py`` (``VisionLayerType`` :53, ``SensitivityReport`` :230).
"""
from __future__ import annotations

import enum
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn as nn

IMAGE_DIR_ENV = {"coco": "MMB200_COCO_DIR", "imagenet": "MMB200_IMAGENET_DIR"}
_IMAGE_EXT = (".jpg", ".jpeg", ".png", ".bmp", ".webp")


@dataclass
class VisionCalibrationConfig:
    dataset: str = "coco"
    num_images: int = 512
    image_size: Tuple[int, int] = (224, 224)
    batch_size: int = 8
    max_batches: Optional[int] = 32
    seed: int = 42
    damping: float = 0.01
    collect_hessians: bool = True
    collect_activations: bool = True


class VisionCalibrationDataset:
    """Float images ``[N, 3, H, W]`` in ``[0, 1]`` with batch iteration."""

    def __init__(self, images: torch.Tensor, name: str = "custom", source: str = "memory"):
        self.images, self.name, self.source = images, name, source

    @property
    def num_images(self) -> int:
        return int(self.images.shape[0])

    @property
    def memory_mb(self) -> float:
        return self.images.numel() * self.images.element_size() / 2 ** 20

    def get_all(self) -> torch.Tensor:
        return self.images

    def get_batches(self, batch_size: int = 8, max_batches: Optional[int] = None) -> Iterator[torch.Tensor]:
        for b, i in enumerate(range(0, self.num_images, batch_size)):
            if max_batches is not None and b >= max_batches:
                return
            yield self.images[i: i + batch_size]

    @classmethod
    def synthetic(cls, num_images: int = 32, image_size: Tuple[int, int] = (224, 224), seed: int = 42) -> "VisionCalibrationDataset":
        """Smooth random fields plus noise (a natural-image-like spectrum rather than white noise), deterministic in ``seed``."""
        g = torch.Generator().manual_seed(seed)
        low = torch.rand(num_images, 3, max(2, image_size[0] // 16), max(2, image_size[1] // 16), generator=g)
        img = torch.nn.functional.interpolate(low, size=tuple(image_size), mode="bicubic", align_corners=False)
        img = img + 0.05 * torch.randn(num_images, 3, *image_size, generator=g)
        return cls(img.clamp_(0, 1), "synthetic", f"seed={seed}")

    @classmethod
    def from_directory(cls, path: str, num_images: int = 512, image_size: Tuple[int, int] = (224, 224), seed: int = 42,
                       name: Optional[str] = None) -> "VisionCalibrationDataset":
        """A seeded sample of the image files below ``path``, decoded with Pillow and resized on this package's preprocessing path."""
        from PIL import Image
        from .device_ops import VisionDevice
        files = sorted(os.path.join(d, f) for d, _, fs in os.walk(path) for f in fs if f.lower().endswith(_IMAGE_EXT))
        if not files:
            raise FileNotFoundError(f"{path}: no image files")
        rng = np.random.RandomState(seed)
        pick = [files[i] for i in sorted(rng.permutation(len(files))[:num_images])]
        vd = VisionDevice("cpu")
        out = [vd.resize_bilinear(torch.from_numpy(np.array(Image.open(p).convert("RGB"))).unsqueeze(0), image_size, nhwc=True)
               .permute(0, 3, 1, 2).float() for p in pick]
        return cls(torch.cat(out), name or os.path.basename(os.path.normpath(path)), path)


def build_vision_calibration_dataset(source: str = "coco", num_images: int = 512, image_size: Tuple[int, int] = (224, 224), seed: int = 42
                                     ) -> VisionCalibrationDataset:
    """``coco`` / ``imagenet``: a sample of the local copy named by ``MMB200_COCO_DIR`` / ``MMB200_IMAGENET_DIR`` (nothing is downloaded);
    a directory path: its images; ``synthetic``: generated images."""
    key = source.lower().replace("_subset", "")
    if key == "synthetic":
        return VisionCalibrationDataset.synthetic(num_images, image_size, seed)
    if key in IMAGE_DIR_ENV:
        d = os.environ.get(IMAGE_DIR_ENV[key])
        if not d or not os.path.isdir(d):
            raise FileNotFoundError(f"{source}: set {IMAGE_DIR_ENV[key]} to a local image directory (there is no download path)")
        return VisionCalibrationDataset.from_directory(d, num_images, image_size, seed, name=key)
    if os.path.isdir(source):
        return VisionCalibrationDataset.from_directory(source, num_images, image_size, seed)
    raise ValueError(f"unsupported calibration dataset source: {source}")


def _is_vision_name(name: str, prefix: str = "") -> bool:
    low = name.lower()
    return bool(prefix and name.startswith(prefix)) or "vision" in low or "visual" in low


def collect_vision_calibration_stats(model: nn.Module, calibration_data: VisionCalibrationDataset, config: Any = None,
                                     forward_fn: Optional[Callable[[Any, Any], Any]] = None, batch_size: int = 8, max_batches: Optional[int] = None,
                                     collect_hessians: bool = True, collect_activations: bool = True, damping: float = 0.01,
                                     max_rows: int = 512) -> Tuple[Dict[str, np.ndarray], Dict[str, np.ndarray]]:
    """Runs the images through ``model`` and returns ``(activations, hessians)`` keyed by weight name (``<module>.weight``) for the
    tower's Linear layers: up to ``max_rows`` input rows per layer, and ``X^T X / n`` with ``damping * mean(diag)`` on the diagonal.
    ``config``: an object with ``layer_prefix`` (only modules under it are hooked), or None for every Linear."""
    prefix = getattr(config, "layer_prefix", "") or ""
    acts: Dict[str, List[torch.Tensor]] = {}
    H: Dict[str, torch.Tensor] = {}
    n: Dict[str, int] = {}
    handles = []

    def make(name):
        def hook(_m, args):
            x = args[0].detach().reshape(-1, args[0].shape[-1]).float()
            if collect_hessians:
                if name not in H:
                    H[name] = torch.zeros(x.shape[1], x.shape[1], device=x.device)
                    n[name] = 0
                H[name].addmm_(x.t(), x)
                n[name] += x.shape[0]
            if collect_activations:
                have = sum(a.shape[0] for a in acts.get(name, []))
                if have < max_rows:
                    acts.setdefault(name, []).append(x[: max_rows - have].cpu())
        return hook

    for name, mod in model.named_modules():
        if isinstance(mod, nn.Linear) and (not prefix or name.startswith(prefix)):
            handles.append(mod.register_forward_pre_hook(make(name + ".weight")))
    try:
        dev = next((p.device for p in model.parameters()), torch.device("cpu"))
        with torch.no_grad():
            for batch in calibration_data.get_batches(batch_size, max_batches):
                batch = batch.to(dev)
                forward_fn(model, batch) if forward_fn is not None else model(batch)
    finally:
        for h in handles:
            h.remove()
    hess = {}
    for k, v in H.items():
        v = v / max(1, n[k])
        v = v + torch.eye(v.shape[0], device=v.device) * damping * torch.diag(v).mean()
        hess[k] = v.cpu().numpy()
    return {k: torch.cat(v).numpy() for k, v in acts.items()}, hess


# ------------------------------------------------------------------------------------------------ sensitivity
class VisionLayerType(str, enum.Enum):
    PATCH_EMBED = "patch_embed"
    POSITION_EMBED = "position_embed"
    CLS_TOKEN = "cls_token"
    LAYER_NORM = "layer_norm"
    ATTENTION_QKV = "attention_qkv"
    ATTENTION_OUT = "attention_out"
    MLP_UP = "mlp_up"
    MLP_DOWN = "mlp_down"
    CROSS_ATTENTION = "cross_attention"
    PROJECTOR = "projector"
    OTHER = "other"


_TYPE_RULES = (
    (("patch_embed", "patch_embedding", "conv1"), VisionLayerType.PATCH_EMBED), (("pos_embed", "position_embedding", "positional"), VisionLayerType.POSITION_EMBED),
    (("cls_token", "class_embedding"), VisionLayerType.CLS_TOKEN), (("norm", "ln_"), VisionLayerType.LAYER_NORM),
    (("cross_attn", "crossattention", "cross_attention"), VisionLayerType.CROSS_ATTENTION), (("projector", "merger", "mm_proj", "multi_modal_projector"), VisionLayerType.PROJECTOR),
    (("qkv", "q_proj", "k_proj", "v_proj", "in_proj"), VisionLayerType.ATTENTION_QKV), (("out_proj", "o_proj", "attn.proj"), VisionLayerType.ATTENTION_OUT),
    (("fc1", "up_proj", "gate_proj", "c_fc"), VisionLayerType.MLP_UP), (("fc2", "down_proj", "c_proj"), VisionLayerType.MLP_DOWN),
)
KEEP_TYPES = (VisionLayerType.PATCH_EMBED, VisionLayerType.POSITION_EMBED, VisionLayerType.LAYER_NORM, VisionLayerType.CLS_TOKEN, VisionLayerType.CROSS_ATTENTION)
# how much an error in a layer of this type matters relative to an MLP matrix
_TYPE_WEIGHT = {VisionLayerType.ATTENTION_QKV: 1.5, VisionLayerType.ATTENTION_OUT: 1.2, VisionLayerType.PROJECTOR: 2.0, VisionLayerType.MLP_UP: 1.0,
                VisionLayerType.MLP_DOWN: 1.1, VisionLayerType.OTHER: 1.0}


def classify_vision_layer(name: str) -> VisionLayerType:
    low = name.lower()
    for frags, t in _TYPE_RULES:
        if any(f in low for f in frags):
            return t
    return VisionLayerType.OTHER


@dataclass
class VisionLayerSensitivity:
    name: str
    layer_type: VisionLayerType
    shape: Tuple[int, ...]
    fp4_error: float
    fp8_error: float
    int4_error: float
    sensitivity_score: float
    recommended_precision: str
    recommended_group_size: int


@dataclass
class SensitivityReport:
    layers: List[VisionLayerSensitivity] = field(default_factory=list)
    fp4_threshold: float = 0.02
    fp8_threshold: float = 0.005

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    def get_by_type(self, layer_type: VisionLayerType) -> List[VisionLayerSensitivity]:
        return [l for l in self.layers if l.layer_type == layer_type]

    def get_precision_summary(self) -> Dict[str, int]:
        out: Dict[str, int] = {}
        for l in self.layers:
            out[l.recommended_precision] = out.get(l.recommended_precision, 0) + 1
        return out

    def estimated_bytes(self) -> float:
        bits = {"fp4": 4.25, "int4": 4.25, "fp8": 8.0, "int8": 8.0, "bf16": 16.0, "fp16": 16.0}
        return sum(float(np.prod(l.shape)) * bits[l.recommended_precision] / 8 for l in self.layers)

    def to_dict(self) -> Dict[str, Any]:
        return {"fp4_threshold": self.fp4_threshold, "fp8_threshold": self.fp8_threshold, "summary": self.get_precision_summary(),
                "layers": [{"name": l.name, "type": l.layer_type.value, "shape": list(l.shape), "fp4_error": l.fp4_error, "fp8_error": l.fp8_error,
                            "int4_error": l.int4_error, "score": l.sensitivity_score, "precision": l.recommended_precision,
                            "group_size": l.recommended_group_size} for l in self.layers]}


def _sim_error(w: torch.Tensor, fmt: str, group_size: int, x: Optional[torch.Tensor], H: Optional[torch.Tensor]) -> float:
    """Relative error of round-to-nearest ``fmt``: in the output ``|| (W - Wq) X^T || / || W X^T ||`` with activations, under
    ``tr(D H D^T) / tr(W H W^T)`` with a Hessian, else in the weights."""
    from ..quant import rtn
    gs = group_size
    while w.shape[1] % gs:
        gs //= 2
    wq = rtn.dequantize(rtn.quantize(w, fmt, max(gs, 8))).float() if w.shape[1] % 8 == 0 else w
    d = w - wq
    if x is not None and x.shape[-1] == w.shape[1]:
        return float((d @ x.t()).norm() / (w @ x.t()).norm().clamp_min(1e-30))
    if H is not None and H.shape[0] == w.shape[1]:
        return float(torch.sqrt(((d @ H) * d).sum().clamp_min(0) / ((w @ H) * w).sum().clamp_min(1e-30)))
    return float(d.norm() / w.norm().clamp_min(1e-30))


def analyze_vision_encoder_sensitivity(weights: Dict[str, Any], activations: Optional[Dict[str, Any]] = None, hessians: Optional[Dict[str, Any]] = None,
                                       fp4_threshold: float = 0.02, fp8_threshold: float = 0.005, group_size: int = 128) -> SensitivityReport:
    """Per matrix: simulated FP4 / INT4 / FP8 error (weighted by the layer type), and the cheapest precision whose weighted
    error is under its threshold — ``fp4`` under ``fp4_threshold``, else ``fp8`` under ``fp8_threshold`` times four (FP8 error is far
    smaller in absolute terms), else ``bf16``; patch / position embeddings, norms, class token and cross attention stay in
    ``bf16`` whatever they measure."""
    rep = SensitivityReport(fp4_threshold=fp4_threshold, fp8_threshold=fp8_threshold)
    for name, w in weights.items():
        w = torch.as_tensor(np.asarray(w) if not isinstance(w, torch.Tensor) else w).float()
        if w.dim() < 2:
            continue
        w2 = w.reshape(w.shape[0], -1)
        t = classify_vision_layer(name)
        x = None if activations is None or name not in activations else torch.as_tensor(np.asarray(activations[name])).float()
        H = None if hessians is None or name not in hessians else torch.as_tensor(np.asarray(hessians[name])).float()
        e4, ei4, e8 = (_sim_error(w2, f, group_size, x, H) for f in ("fp4", "int4", "fp8"))
        score = e4 * _TYPE_WEIGHT.get(t, 1.0)
        if t in KEEP_TYPES:
            prec, gs = "bf16", 0
        elif score <= fp4_threshold:
            prec, gs = "fp4", group_size
        elif score <= 2 * fp4_threshold:
            prec, gs = "fp4", max(32, group_size // 2)            # a finer group first
        elif e8 * _TYPE_WEIGHT.get(t, 1.0) <= 4 * fp8_threshold:
            prec, gs = "fp8", group_size
        else:
            prec, gs = "bf16", 0
        rep.layers.append(VisionLayerSensitivity(name, t, tuple(w.shape), e4, e8, ei4, score, prec, gs))
    return rep


def _precision(value):
    from ..compat_api import Precision
    return value if isinstance(value, Precision) else Precision(str(value).lower().replace("fp4_e2m1", "fp4").replace("fp8_e4m3", "fp8"))


def _default_vision_precision(name: str, config: Any) -> Tuple[str, int]:
    if config is not None and hasattr(config, "get_layer_precision"):
        return config.get_layer_precision(name)
    if config is not None and hasattr(config, "should_quantize"):        # vision.VisionQuantConfig
        return (config.fmt, config.group_size) if config.should_quantize(name, (64, 64)) else ("bf16", 0)
    return ("bf16", 0) if classify_vision_layer(name) in KEEP_TYPES + (VisionLayerType.PROJECTOR,) else ("fp8", 128)


def build_vision_precision_map(weights: Dict[str, Any], config: Any = None, report: Optional[SensitivityReport] = None) -> Dict[str, Tuple[Any, int]]:
    """``{weight name: (Precision, group size)}`` for the matrices of the tower: the report's recommendation when there is one
    (never below 16 bits for the keep-types), else the configuration's default for that layer."""
    by_name = {l.name: l for l in report.layers} if report is not None else {}
    out = {}
    for name, w in weights.items():
        if np.ndim(w) < 2:
            continue
        l = by_name.get(name)
        if l is not None:
            out[name] = (_precision("bf16"), 0) if l.layer_type in KEEP_TYPES else (_precision(l.recommended_precision), l.recommended_group_size)
        else:
            p, gs = _default_vision_precision(name, config)
            out[name] = (_precision(p), gs)
    return out


def build_vlm_precision_map(weights: Dict[str, Any], vision_config: Any = None, vision_precision_map: Optional[Dict[str, Tuple[Any, int]]] = None,
                            llm_precision: Any = "fp4", llm_group_size: int = 128, keep_llm_sensitive: bool = True) -> Dict[str, Tuple[Any, int]]:
    """The whole model: tower matrices from ``vision_precision_map`` (or the tower default), language-model matrices in
    ``llm_precision`` — embeddings, norms and the output head in ``bf16`` when ``keep_llm_sensitive``."""
    vmap = vision_precision_map or {}
    prefix = getattr(vision_config, "layer_prefix", "") or ""
    out = {}
    for name, w in weights.items():
        if np.ndim(w) < 2:
            continue
        low = name.lower()
        if name in vmap:
            out[name] = vmap[name]
        elif _is_vision_name(name, prefix):
            p, gs = _default_vision_precision(name, vision_config)
            out[name] = (_precision(p), gs)
        elif keep_llm_sensitive and any(f in low for f in ("embed", "norm", "lm_head", "output")):
            out[name] = (_precision("bf16"), 0)
        else:
            out[name] = (_precision(llm_precision), llm_group_size)
    return out


def pack_vlm_mixed_format(weights: Dict[str, Any], precision_map: Dict[str, Tuple[Any, int]], output_path: str):
    """Quantize every tensor to its mapped precision into one mixed-format file; tensors without an entry (vectors) are kept in
    16 bits.  Returns the pack."""
    from ..converters.mixed_format import build_mixed_pack
    pack = build_mixed_pack(weights, precision_map)
    pack.save(output_path)
    return pack
