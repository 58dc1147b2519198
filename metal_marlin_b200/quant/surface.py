"""The reference's ``metal_marlin.quantization`` and ``metal_marlin.calibration`` names on this package's quantizers: the
EXL3-style quantizer objects and pipeline (Hessian preprocessing, block rotation, LDL feedback, tile scales), layer
streaming over a checkpoint, calibration datasets / hooks, and sensitivity profiles with a recommendation step.

Parity: reference ``quantization/__init__.py`` (``EXL3Quantizer`` / ``EXL3QuantResult`` / ``EXL3QuantizerPipeline``, ``ldlq_quantize_layer``,
``ldl_solve``, ``preprocess_hessian_exl3``, ``rotate_weights_exl3`` / ``unrotate_weights_exl3``, ``blockwise_hadamard``, ``compute_tile_scales``,
``quantize_tiles_parallel``, ``TrellisCodebook`` / ``TrellisTile``, ``tensor_core_perm*``, ``LayerStreamer`` / ``LayerInfo`` / ``LayerWeights``,
``StreamingQuantizer`` / ``quantize_model_streaming``, ``CalibrationStreamer`` / ``CalibrationBatch``, ``StreamingHessianCollector``,
``collect_layer_hessian`` / ``collect_all_hessians_streaming``, ``copy_non_linear_tensors``, ``save_exl3_layer``, ``quantize_model_exl3``) and
``calibration/__init__.py`` (``BartowskiCalibration``, ``CalibrationDataset``, ``CalibrationHooks`` / ``GQACalibrationHooks``,
``analyze_layer_sensitivity``, ``compute_model_sensitivity_profile``, ``save_`` / ``load_sensitivity_profile``, ``recommend_quantization``,
``sensitivity_to_config``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence, Tuple

import torch

from . import hadamard as _had
from . import ldlq as _ldlq
from .calibration import KNOWN_DATASETS, HessianCollector, load_calibration_tokens
from .mixed_precision import allocate_bits

_HAS_SAFETENSORS = True          # own safetensors reader / writer
_HAS_STREAMING = True
try:
    import transformers as _tf      # noqa: F401
    _HAS_TRANSFORMERS = True
except Exception:                    # pragma: no cover
    _HAS_TRANSFORMERS = False

StreamingHessianCollector = HessianCollector


# ------------------------------------------------------------------------------------------------ EXL3-style pieces
def blockwise_hadamard(x: torch.Tensor, block: int = 128) -> torch.Tensor:
    return _had.block_hadamard(x, block)


def rotate_weights_exl3(w: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Input-side block-Hadamard rotation of ``w [out, in]`` (``in`` a multiple of ``block``)."""
    return _had.rotate_weight(w, block)


def unrotate_weights_exl3(w: torch.Tensor, block: int = 128) -> torch.Tensor:
    """The orthonormal block transform is an involution."""
    return _had.rotate_weight(w, block)


def preprocess_hessian_exl3(H: torch.Tensor, damp: float = 0.01, block: int = 0) -> torch.Tensor:
    """Symmetrise, give dead inputs a unit diagonal, damp by ``damp * mean(diag)`` and (with ``block``) rotate into the basis of
    block-Hadamard-rotated weights."""
    H = 0.5 * (H.float() + H.float().t())
    dead = torch.diag(H) <= 0
    H[dead, dead] = 1.0
    H = H + torch.eye(H.shape[0], device=H.device) * damp * torch.diag(H).mean()
    return _had.rotate_hessian(H, block) if block else H


def ldl_solve(H: torch.Tensor, block: int = 16, damp: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Block LDL factorisation ``H = L D L^T`` (unit block-lower ``L`` minus the identity is the feedback matrix)."""
    return _ldlq.block_ldl(H, block, damp)


def compute_tile_scales(w: torch.Tensor, bits: int, group_size: int = 128) -> torch.Tensor:
    return _ldlq.compute_group_scales(w, bits, group_size)


def quantize_tiles_parallel(tiles: torch.Tensor, scales: torch.Tensor, bits: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """All rows of a column block at once: ``tiles [out, 16]`` with ``scales [out, 1]`` -> ``(codes, de-quantized)``."""
    return _ldlq.quantize_tile_greedy(tiles, scales, bits)


def compute_quantization_error(w: torch.Tensor, wq: torch.Tensor, H: Optional[torch.Tensor] = None) -> Dict[str, float]:
    d = (w.float() - wq.float())
    out = {"mse": float(d.pow(2).mean()), "relative": float(d.norm() / w.float().norm().clamp_min(1e-30)), "max_abs": float(d.abs().max())}
    if H is not None:
        out["proxy"] = _ldlq.proxy_error(w.double(), wq.double(), H.double())
    return out


@dataclass
class TrellisTile:
    row: int
    col: int
    codes: torch.Tensor            # uint8 [16, 16]
    bits: int


class TrellisCodebook:
    """The uniform grid of a bit width: ``values`` (2**bits levels, symmetric, unit spread constant of the format) with
    nearest-level ``encode`` and ``decode``."""

    def __init__(self, bits: int, device="cpu"):
        from ..formats.trellis import trellis_grid
        self.bits = bits
        self.values = trellis_grid(bits, device)

    def encode(self, x: torch.Tensor) -> torch.Tensor:
        mids = (self.values[1:] + self.values[:-1]) / 2
        return torch.bucketize(x.float(), mids).to(torch.uint8)

    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        return self.values[codes.long()]


def tensor_core_perm(device="cpu") -> torch.Tensor:
    """Order in which the 256 values of a 16 x 16 tile are laid out for an m16n8k16-style fragment load: thread ``t`` of a
    warp owns rows ``t / 4`` and ``t / 4 + 8``, column pairs ``2 (t % 4)`` and ``2 (t % 4) + 8``."""
    idx = []
    for t in range(32):
        r, c = t // 4, 2 * (t % 4)
        for rr, cc in ((r, c), (r + 8, c), (r, c + 8), (r + 8, c + 8)):
            idx += [rr * 16 + cc, rr * 16 + cc + 1]
    return torch.tensor(idx, dtype=torch.long, device=device)


def tensor_core_perm_i(device="cpu") -> torch.Tensor:
    p = tensor_core_perm(device)
    inv = torch.empty_like(p)
    inv[p] = torch.arange(256, device=p.device)
    return inv


def apply_tensor_core_perm(tile: torch.Tensor) -> torch.Tensor:
    """``[..., 16, 16] -> [..., 256]`` in fragment order."""
    return tile.reshape(*tile.shape[:-2], 256)[..., tensor_core_perm(tile.device)]


def apply_tensor_core_perm_i(flat: torch.Tensor) -> torch.Tensor:
    return flat[..., tensor_core_perm_i(flat.device)].reshape(*flat.shape[:-1], 16, 16)


@dataclass
class EXL3QuantResult:
    weight: Any                    # formats.trellis.TrellisWeight
    dequantized: torch.Tensor
    proxy_error: float
    mse: float
    bits: int


QuantizationResult = EXL3QuantResult


def ldlq_quantize_layer(w: torch.Tensor, H: Optional[torch.Tensor], bits: int = 4, group_size: int = 128, **kw) -> EXL3QuantResult:
    r = _ldlq.ldlq_quantize(w, H, bits, group_size, **kw)
    return EXL3QuantResult(r.weight, r.dequantized, r.proxy_error, r.mse, bits)


ldlq_quantize_layer_core = ldlq_quantize_layer


class EXL3Quantizer:
    def __init__(self, bits: int = 4, group_size: int = 128, damp: float = 0.01):
        self.bits, self.group_size, self.damp = bits, group_size, damp

    def quantize_layer(self, w: torch.Tensor, H: Optional[torch.Tensor] = None) -> EXL3QuantResult:
        return ldlq_quantize_layer(w, H, self.bits, self.group_size, damp=self.damp)


def quantize_model_exl3(model_dir: str, out_dir: str, bits: int = 4, group_size: int = 128, calibration: str = "synthetic",
                        num_samples: int = 32, seq_len: int = 512, target_bpw: Optional[float] = None, device: Optional[str] = None) -> dict:
    """Whole-checkpoint EXL3-style quantization (calibration Hessians, LDL feedback, optional mixed bit widths)."""
    from .pipeline import quantize_checkpoint
    return quantize_checkpoint(model_dir, out_dir, fmt="trellis-v2", method="ldlq", group_size=group_size, bits=bits, calibration=calibration,
                               num_samples=num_samples, seq_len=seq_len, target_bpw=target_bpw, device=device)


class EXL3QuantizerPipeline:
    def __init__(self, bits: int = 4, group_size: int = 128, calibration: str = "synthetic", num_samples: int = 32, seq_len: int = 512,
                 target_bpw: Optional[float] = None):
        self.kw = dict(bits=bits, group_size=group_size, calibration=calibration, num_samples=num_samples, seq_len=seq_len, target_bpw=target_bpw)

    def run(self, model_dir: str, out_dir: str, device: Optional[str] = None) -> dict:
        return quantize_model_exl3(model_dir, out_dir, device=device, **self.kw)


def save_exl3_layer(weights: Dict[str, Any], out_dir: str, layer_index: int) -> str:
    """One layer of trellis weights in the layer-directory container (``layer_NNNN/index.json`` + tensor files)."""
    from ..formats.safetensors_io import save_file
    from ..formats.trellis import SUFFIXES, tensor_key
    d = os.path.join(out_dir, f"layer_{layer_index:04d}")
    os.makedirs(d, exist_ok=True)
    entries = []
    for j, (name, tw) in enumerate(weights.items()):
        save_file({tensor_key(name, p): getattr(tw, p) for p in SUFFIXES}, os.path.join(d, f"tensor_{j:04d}.safetensors"))
        entries.append({"name": name, "bits": tw.bits, "shape": list(tw.shape), "mse": 0.0})
    with open(os.path.join(d, "index.json"), "w") as f:
        json.dump({"tensors": entries}, f)
    return d


# ------------------------------------------------------------------------------------------------ layer streaming
@dataclass
class LayerInfo:
    index: int
    tensor_names: List[str]
    nbytes: int


@dataclass
class LayerWeights:
    index: int
    tensors: Dict[str, torch.Tensor]


class LayerStreamerBase:
    def __iter__(self) -> Iterator[LayerWeights]:
        raise NotImplementedError


class LayerStreamer(LayerStreamerBase):
    """Decoder layers of a checkpoint one at a time (the next layer is read by a background thread meanwhile), so a model
    larger than host memory can be processed."""

    def __init__(self, model_dir: str, device=None):
        from ..formats.mmfp4_loader import MMFP4ModelLoader
        self.loader = MMFP4ModelLoader(model_dir, prefetch_workers=1)
        self.device = device

    def layer_infos(self) -> List[LayerInfo]:
        out = []
        for i in range(self.loader.num_layers()):
            names = self.loader.layer_tensor_names(i)
            nb = 0
            for n in names:
                f = self.loader._file(self.loader.weight_map[n])
                nb += int(torch.tensor(f.shape(n)).prod()) * {"F32": 4, "I32": 4, "U32": 4, "F16": 2, "BF16": 2}.get(f.dtype_str(n), 1)
            out.append(LayerInfo(i, names, nb))
        return out

    def non_layer_tensors(self) -> Dict[str, torch.Tensor]:
        from ..formats.mmfp4_loader import extract_layer_index
        return {k: self.loader.load_tensor(k) for k in self.loader.tensor_names() if extract_layer_index(k) is None}

    def __iter__(self) -> Iterator[LayerWeights]:
        n = self.loader.num_layers()
        for i in range(n):
            if i + 1 < n:
                self.loader.prefetch_layer(i + 1)
            yield LayerWeights(i, self.loader.load_layer(i, self.device))


def copy_non_linear_tensors(model_dir: str, out_file: str) -> int:
    """Everything quantization leaves alone (embeddings, norms, router gates, biases) into one file; returns the count."""
    from ..checkpoint_tools import extract_base_weights
    return extract_base_weights(model_dir, out_file)["tensors"]


@dataclass
class StreamingQuantResult:
    layers: int
    tensors: int
    info: dict = field(default_factory=dict)


class StreamingQuantizer:
    """Layer-by-layer quantization of a checkpoint through the offline pipeline (tensors are read, quantized and written
    shard by shard; nothing but the current tensors is held)."""

    def __init__(self, fmt: str = "mmfp4", method: str = "rtn", group_size: int = 128, **kw):
        self.fmt, self.method, self.group_size, self.kw = fmt, method, group_size, kw

    def quantize(self, model_dir: str, out_dir: str, device: Optional[str] = None) -> StreamingQuantResult:
        from .pipeline import quantize_checkpoint
        info = quantize_checkpoint(model_dir, out_dir, fmt=self.fmt, method=self.method, group_size=self.group_size, device=device, **self.kw)
        from ..formats.mmfp4_loader import MMFP4ModelLoader
        try:
            n_layers = MMFP4ModelLoader(out_dir, prefetch_workers=0).num_layers()
        except Exception:
            n_layers = 0
        return StreamingQuantResult(n_layers, int(info.get("quantized", 0)), info)


def quantize_model_streaming(model_dir: str, out_dir: str, fmt: str = "mmfp4", method: str = "rtn", group_size: int = 128, **kw) -> StreamingQuantResult:
    return StreamingQuantizer(fmt, method, group_size, **kw).quantize(model_dir, out_dir)


# ------------------------------------------------------------------------------------------------ calibration data and hooks
@dataclass
class CalibrationBatch:
    input_ids: torch.Tensor        # [B, T]
    index: int


class CalibrationDataset:
    """Token sequences for calibration: a named set (``bartowski-v3`` / ``wikitext2`` / ``c4`` resolved to local text when present,
    a deterministic synthetic stream otherwise) or a text file."""

    def __init__(self, name: str = "synthetic", tokenizer=None, vocab_size: int = 32000, num_samples: int = 32, seq_len: int = 512, seed: int = 0):
        self.name = name
        self.samples = load_calibration_tokens(name, tokenizer, vocab_size, num_samples, seq_len, seed)

    def __len__(self) -> int:
        return len(self.samples)

    def __getitem__(self, i: int) -> List[int]:
        return self.samples[i]

    def __iter__(self):
        return iter(self.samples)


class BartowskiCalibration(CalibrationDataset):
    def __init__(self, tokenizer=None, vocab_size: int = 32000, num_samples: int = 32, seq_len: int = 512, seed: int = 0):
        super().__init__("bartowski-v3", tokenizer, vocab_size, num_samples, seq_len, seed)


BartowskiCalibrationV3 = BartowskiCalibration


class CalibrationStreamer:
    """Batches of a calibration set as tensors."""

    def __init__(self, dataset: CalibrationDataset, batch_size: int = 4):
        self.dataset, self.batch_size = dataset, batch_size

    def __iter__(self) -> Iterator[CalibrationBatch]:
        s = self.dataset.samples
        for i in range(0, len(s), self.batch_size):
            yield CalibrationBatch(torch.tensor(s[i: i + self.batch_size], dtype=torch.int64), i // self.batch_size)


class CalibrationHooks:
    """Context manager that records the inputs of every quantizable projection of the engine's models while they run
    (``with CalibrationHooks() as h: lm.forward_logits(ids)``; afterwards ``h.collector`` holds one Hessian per checkpoint
    tensor name, per expert for MoE banks)."""

    def __init__(self, collector: Optional[HessianCollector] = None):
        self.collector = collector or HessianCollector()

    def _hook(self, kind, W, x, ids):
        if getattr(W, "names", None) is None:
            return
        if kind == "linear":
            for name, _rows in W.names:
                self.collector.add(name, x)
            return
        flat = x.reshape(-1, x.shape[-1]) if kind == "moe_down" else None
        for e in ids.unique().tolist():
            if e < 0 or e >= len(W.names):
                continue
            rows = x[(ids == e).any(1)] if kind == "moe_gate_up" else flat[(ids == e).reshape(-1)]
            for name, _rows in W.names[e]:
                self.collector.add(name, rows)

    def __enter__(self):
        from .. import ops
        ops.set_capture(self._hook)
        return self

    def __exit__(self, *exc):
        from .. import ops
        ops.set_capture(None)
        return False


GQACalibrationHooks = CalibrationHooks      # fused q | k | v matrices share one input: the hook feeds each of their tensor names


def collect_layer_hessian(activations: torch.Tensor, normalize: bool = True) -> torch.Tensor:
    x = activations.reshape(-1, activations.shape[-1]).float()
    H = x.t() @ x
    return H / max(1, x.shape[0]) if normalize else H


def collect_all_hessians_streaming(model_dir_fp4: str, calibration: str = "synthetic", num_samples: int = 32, seq_len: int = 512,
                                   device: Optional[str] = None) -> HessianCollector:
    from .pipeline import collect_hessians
    return collect_hessians(model_dir_fp4, calibration, num_samples, seq_len, device)


# ------------------------------------------------------------------------------------------------ sensitivity
def analyze_layer_sensitivity(w: torch.Tensor, H: Optional[torch.Tensor] = None, bit_choices: Sequence[int] = (2, 3, 4, 5, 6, 8),
                              group_size: int = 128) -> Dict[int, float]:
    """Error of nearest-grid trellis quantization of ``w`` at every candidate bit width, under the Hessian metric when ``H``
    is given (relative squared error otherwise)."""
    from ..formats.trellis import quantize_trellis
    out = {}
    for b in bit_choices:
        wq = quantize_trellis(w.float(), b, group_size).dequantize(torch.float32)
        if H is not None:
            out[int(b)] = _ldlq.proxy_error(w.double(), wq.double(), H.double())
        else:
            out[int(b)] = float(((w.float() - wq) ** 2).sum() / (w.float() ** 2).sum().clamp_min(1e-30))
    return out


def compute_model_sensitivity_profile(tensors: Dict[str, torch.Tensor], hessians: Optional[Dict[str, torch.Tensor]] = None,
                                      bit_choices: Sequence[int] = (2, 3, 4, 5, 6, 8), group_size: int = 128) -> Dict[str, Dict]:
    prof = {}
    for name, w in tensors.items():
        H = None if hessians is None else hessians.get(name)
        prof[name] = {"num_params": int(w.numel()), "error_by_bits": analyze_layer_sensitivity(w, H, bit_choices, group_size)}
    return prof


def save_sensitivity_profile(profile: Dict[str, Dict], path: str) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        json.dump({k: {"num_params": v["num_params"], "error_by_bits": {str(b): e for b, e in v["error_by_bits"].items()}}
                   for k, v in profile.items()}, f, indent=1)


def load_sensitivity_profile(path: str) -> Dict[str, Dict]:
    with open(path) as f:
        d = json.load(f)
    return {k: {"num_params": v["num_params"], "error_by_bits": {int(b): e for b, e in v["error_by_bits"].items()}} for k, v in d.items()}


def recommend_quantization(profile: Dict[str, Dict], target_bpw: float = 4.0) -> Dict[str, int]:
    """Bit width per tensor: the greedy marginal-gain allocation under the average bits-per-weight target."""
    sens = {k: v["error_by_bits"] for k, v in profile.items()}
    sizes = {k: v["num_params"] for k, v in profile.items()}
    choices = sorted({b for v in sens.values() for b in v})
    return allocate_bits(sens, sizes, target_bpw, choices)


def sensitivity_to_config(profile: Dict[str, Dict], target_bpw: float = 4.0, group_size: int = 128) -> Dict[str, Dict]:
    """``{tensor name: {"bits", "group_size", "format"}}`` for the quantization driver (``bit_allocation`` of the trellis writer)."""
    return {k: {"bits": b, "group_size": group_size, "format": "trellis"} for k, b in recommend_quantization(profile, target_bpw).items()}


# ------------------------------------------------------------------------------------------------ trellis search, config, Hessian manager
def quantize_tile_viterbi(tile: torch.Tensor, codebook: TrellisCodebook, scale: float, transition_penalty: float = 0.0
                          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Minimum-cost path through the level trellis of a tile (flattened row by row): cost ``sum_i (x_i / scale - g[s_i])^2 +
    transition_penalty * sum_i |s_i - s_{i-1}|``.  With no transition penalty every element takes its nearest level; a positive one
    trades a little error for smoother index sequences.  Returns ``(indices uint8 [n], de-quantized tile)``.
    Reference ``quantization/viterbi_quant.py:91``."""
    g = codebook.values.to(torch.float64)
    x = tile.reshape(-1).to(torch.float64) / float(scale)
    n, S = x.numel(), g.numel()
    local = (x[:, None] - g[None, :]) ** 2                                        # [n, S]
    if transition_penalty <= 0.0:
        idx = local.argmin(1)
    else:
        states = torch.arange(S, dtype=torch.float64)
        trans = transition_penalty * (states[:, None] - states[None, :]).abs()   # [prev, cur]
        cost = local[0].clone()
        back = torch.zeros(n, S, dtype=torch.long)
        for i in range(1, n):
            total = cost[:, None] + trans
            cost, back[i] = total.min(0)
            cost = cost + local[i]
        idx = torch.empty(n, dtype=torch.long)
        idx[-1] = int(cost.argmin())
        for i in range(n - 1, 0, -1):
            idx[i - 1] = back[i, idx[i]]
    deq = (g[idx] * float(scale)).to(tile.dtype).reshape(tile.shape)
    return idx.to(torch.uint8), deq


def write_exl3_config(output_path: str, bits: int, group_size: int, results: Sequence[EXL3QuantResult]) -> str:
    """``quantization_config.json`` in ``output_path``: method, bit width, group size, and the summary of the layer results."""
    os.makedirs(str(output_path), exist_ok=True)
    n = max(1, len(results))
    cfg = {"quantization_config": {"quant_method": "exl3", "bits": int(bits), "group_size": int(group_size), "format": f"exl3_{int(bits)}bit",
                                   "symmetric": True, "desc_act": False},
           "quantization_stats": {"layers_quantized": len(results), "avg_reconstruction_mse": sum(float(r.mse) for r in results) / n,
                                  "avg_proxy_error": sum(float(r.proxy_error) for r in results) / n,
                                  "bits_histogram": {str(b): sum(1 for r in results if r.bits == b) for b in sorted({r.bits for r in results})}}}
    path = os.path.join(str(output_path), "quantization_config.json")
    with open(path, "w") as f:
        json.dump(cfg, f, indent=1)
    return path


class HessianManager:
    """Named Hessian accumulators with explicit registration: ``register_layer(name, in_features)``, ``accumulate_layer(name, x)``,
    ``get_hessian(name, damp)`` (mean of ``x x^T`` plus ``damp * mean(diag)`` on the diagonal).  ``attach(module)`` registers every
    ``nn.Linear`` below a module and hooks its input.  Reference ``calibration/hessian_collector.py:218``."""

    def __init__(self, default_damp: float = 0.01):
        self.default_damp = default_damp
        self._dims: Dict[str, int] = {}
        self._col = HessianCollector()
        self._handles: list = []

    def register_layer(self, name: str, in_features: int) -> None:
        if name in self._dims and self._dims[name] != in_features:
            raise ValueError(f"{name} is registered with {self._dims[name]} input features")
        self._dims[name] = int(in_features)

    def unregister_layer(self, name: str) -> None:
        self._dims.pop(name, None)
        self.reset_layer(name)

    def accumulate_layer(self, name: str, x) -> None:
        if name not in self._dims:
            raise KeyError(f"layer {name!r} is not registered")
        x = torch.as_tensor(x)
        if x.shape[-1] != self._dims[name]:
            raise ValueError(f"{name}: activations have {x.shape[-1]} features, registered {self._dims[name]}")
        self._col.add(name, x)

    def get_hessian(self, name: str, damp: Optional[float] = None) -> torch.Tensor:
        if name not in self._dims:
            raise KeyError(f"layer {name!r} is not registered")
        H = self._col.get(name)
        if H is None:
            H = torch.zeros(self._dims[name], self._dims[name])
        damp = self.default_damp if damp is None else damp
        level = torch.diag(H).mean() if float(torch.diag(H).mean()) > 0 else torch.tensor(1.0)
        return H + torch.eye(H.shape[0], device=H.device) * damp * level

    def get_all_hessians(self, damp: Optional[float] = None) -> Dict[str, torch.Tensor]:
        return {n: self.get_hessian(n, damp) for n in self._dims}

    def get_sample_counts(self) -> Dict[str, int]:
        return {n: int(self._col.n.get(n, 0)) for n in self._dims}

    def reset_layer(self, name: str) -> None:
        self._col.H.pop(name, None)
        self._col.n.pop(name, None)

    def reset_all(self) -> None:
        self._col.H.clear()
        self._col.n.clear()

    def attach(self, module, prefix: str = "") -> int:
        import torch.nn as nn
        count = 0
        for name, m in module.named_modules():
            if isinstance(m, nn.Linear):
                full = f"{prefix}{name}"
                self.register_layer(full, m.in_features)
                self._handles.append(m.register_forward_pre_hook(lambda _m, args, _n=full: self.accumulate_layer(_n, args[0].detach())))
                count += 1
        return count

    def remove_hooks(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []

    @property
    def layer_names(self) -> List[str]:
        return list(self._dims)

    @property
    def num_layers(self) -> int:
        return len(self._dims)
