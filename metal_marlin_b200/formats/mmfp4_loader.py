"""Loader for quantized checkpoints in the ``mmfp4`` and ``marlin_fp4`` layouts.

Accepts a directory with ``model.safetensors.index.json`` + shards or a single
``model.safetensors``; resolves HF tensor-name variants (``model.language_model.`` <->
``model.``), weight/scale key aliases, per-layer loading, streaming iteration and a
background prefetcher.

Parity: reference ``metal_marlin/mmfp4_loader.py:378`` (``MMFP4ModelLoader``): ``_parse_index``
``:431``, raw header parse ``:521``, ``_extract_layer_index`` ``:540``, ``_generate_name_variants``
``:561``, ``load_tensor`` ``:625``, ``load_layer`` ``:1037``, ``get_quantized_weight`` ``:1248``
(suffix aliases ``:1264-1265``), ``WeightPrefetcher`` ``:81``.
"""
from __future__ import annotations

import json
import os
import re
import threading
from collections import OrderedDict
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Dict, Iterator, List, Optional, Tuple

import torch

from .safetensors_io import SafetensorsFile

WEIGHT_SUFFIXES = (".qweight", ".weight", ".packed_weight")      # probe order of the reference loader
SCALE_SUFFIXES = (".scales", ".weight_scale", ".scales_fp4", ".weight.scales")
_LAYER_RE = re.compile(r"(?:layers|h|blocks)\.(\d+)\.")


def extract_layer_index(name: str) -> Optional[int]:
    m = _LAYER_RE.search(name)
    return int(m.group(1)) if m else None


def name_variants(name: str) -> List[str]:
    out = [name]
    if name.startswith("model.language_model."):
        out.append("model." + name[len("model.language_model."):])
        out.append(name[len("model."):])
    elif name.startswith("language_model.model."):
        out.append(name[len("language_model."):])
    elif name.startswith("model."):
        out.append("model.language_model." + name[len("model."):])
        out.append("language_model." + name)
    else:
        out.append("model." + name)
    return out


class MMFP4ModelLoader:
    def __init__(self, path: str, prefetch_workers: int = 2, cache_files: int = 8):
        self.path = path
        self.weight_map: Dict[str, str] = {}
        self._files: "OrderedDict[str, SafetensorsFile]" = OrderedDict()
        self._cache_files = cache_files
        self._lock = threading.Lock()
        self._pool = ThreadPoolExecutor(max_workers=prefetch_workers) if prefetch_workers else None
        self._prefetched: Dict[int, Future] = {}
        self.quant_config: dict = {}
        self._parse_index()

    # ------------------------------------------------------------------ index
    def _parse_index(self) -> None:
        idx = os.path.join(self.path, "model.safetensors.index.json")
        single = os.path.join(self.path, "model.safetensors")
        if os.path.isfile(self.path) and self.path.endswith(".safetensors"):
            single, self.path = self.path, os.path.dirname(self.path)
        if os.path.exists(idx):
            with open(idx) as f:
                self.weight_map = dict(json.load(f)["weight_map"])
        elif os.path.exists(single):
            with SafetensorsFile(single) as f:
                self.weight_map = {k: os.path.basename(single) for k in f.keys()}
        else:
            shards = sorted(f for f in os.listdir(self.path) if f.endswith(".safetensors"))
            if not shards:
                raise FileNotFoundError(f"no safetensors checkpoint under {self.path}")
            for s in shards:
                with SafetensorsFile(os.path.join(self.path, s)) as f:
                    for k in f.keys():
                        self.weight_map[k] = s
        for cand in ("quantization_config.json",):
            p = os.path.join(self.path, cand)
            if os.path.exists(p):
                with open(p) as f:
                    self.quant_config = json.load(f)
        if not self.quant_config:
            cfgp = os.path.join(self.path, "config.json")
            if os.path.exists(cfgp):
                with open(cfgp) as f:
                    self.quant_config = json.load(f).get("quantization_config", {}) or {}

    @property
    def format(self) -> str:
        fmt = str(self.quant_config.get("format", "")).lower()
        if "marlin_fp4" in fmt:
            return "marlin_fp4"
        return "mmfp4"

    def _file(self, fname: str) -> SafetensorsFile:
        with self._lock:
            f = self._files.get(fname)
            if f is None:
                f = SafetensorsFile(os.path.join(self.path, fname))
                self._files[fname] = f
                while len(self._files) > self._cache_files:
                    _, old = self._files.popitem(last=False)
                    old.close()
            else:
                self._files.move_to_end(fname)
            return f

    # ------------------------------------------------------------------ lookup
    def resolve(self, name: str) -> Optional[str]:
        for v in name_variants(name):
            if v in self.weight_map:
                return v
        return None

    def has_tensor(self, name: str) -> bool:
        return self.resolve(name) is not None

    def tensor_names(self) -> List[str]:
        return list(self.weight_map.keys())

    def load_tensor(self, name: str) -> torch.Tensor:
        key = self.resolve(name)
        if key is None:
            raise KeyError(f"tensor {name!r} not found (tried {name_variants(name)})")
        return self._file(self.weight_map[key]).get_tensor(key)

    def _find(self, base: str, suffixes) -> Optional[str]:
        for s in suffixes:
            k = self.resolve(base + s)
            if k is not None:
                return k
        return None

    def is_quantized(self, base: str) -> bool:
        """``base`` is a module path without suffix (e.g. ``model.layers.0.self_attn.o_proj``)."""
        w = self._find(base, WEIGHT_SUFFIXES)
        s = self._find(base, SCALE_SUFFIXES)
        if w is None or s is None:
            return False
        dt = self._file(self.weight_map[w]).dtype_str(w)
        return dt in ("U32", "I32")

    def get_quantized_weight(self, base: str) -> Tuple[torch.Tensor, torch.Tensor, str]:
        """Returns ``(packed int32, scales fp16, layout)``; layout is ``"mmfp4"`` (row packed
        ``[out, in/8]``) or ``"marlin_fp4"`` (``[in/8, out]``)."""
        w = self._find(base, WEIGHT_SUFFIXES)
        s = self._find(base, SCALE_SUFFIXES)
        if w is None or s is None:
            raise KeyError(f"no quantized weight for {base!r}")
        packed = self._file(self.weight_map[w]).get_tensor(w)
        scales = self._file(self.weight_map[s]).get_tensor(s)
        return packed, scales.to(torch.float16), self.format

    def get_group_size(self, base: str, default: int = 128) -> int:
        k = self._find(base, (".group_size", ".weight.group_size"))
        if k is not None:
            return int(self._file(self.weight_map[k]).get_tensor(k).reshape(-1)[0])
        return int(self.quant_config.get("group_size", default))

    def get_hadamard_block_size(self, base: str) -> int:
        k = self._find(base, (".hadamard_block_size", ".weight.hadamard_block_size"))
        return int(self._file(self.weight_map[k]).get_tensor(k).reshape(-1)[0]) if k else 0

    # ------------------------------------------------------------------ bulk access
    def layer_tensor_names(self, layer: int) -> List[str]:
        return [k for k in self.weight_map if extract_layer_index(k) == layer]

    def load_layer(self, layer: int, device=None) -> Dict[str, torch.Tensor]:
        fut = self._prefetched.pop(layer, None)
        out = fut.result() if fut is not None else {k: self.load_tensor(k) for k in self.layer_tensor_names(layer)}
        if device is not None:
            out = {k: v.to(device, non_blocking=True) for k, v in out.items()}
        return out

    def prefetch_layer(self, layer: int) -> None:
        if self._pool is None or layer in self._prefetched:
            return
        names = self.layer_tensor_names(layer)
        self._prefetched[layer] = self._pool.submit(lambda: {k: self.load_tensor(k) for k in names})

    def stream_weights(self) -> Iterator[Tuple[str, torch.Tensor]]:
        for k in self.weight_map:
            yield k, self.load_tensor(k)

    def num_layers(self) -> int:
        idx = [extract_layer_index(k) for k in self.weight_map]
        idx = [i for i in idx if i is not None]
        return max(idx) + 1 if idx else 0

    def close(self) -> None:
        for f in self._files.values():
            f.close()
        self._files.clear()
        if self._pool is not None:
            self._pool.shutdown(wait=False)
