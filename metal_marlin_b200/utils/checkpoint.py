"""Checkpoint utilities: load (single / sharded / lazy), save, key remapping and filtering.

Parity: reference ``metal_marlin/checkpoint.py`` — ``load_checkpoint`` ``:95``, ``load_sharded_checkpoint`` ``:134``,
``LazyCheckpoint`` ``:287``, ``save_checkpoint`` ``:430``, ``remap_weight_keys`` ``:452``, ``filter_weights`` ``:509``.
"""
from __future__ import annotations

import json
import os
import re
from typing import Callable, Dict, Iterable, Iterator, List, Optional

import torch

from ..formats.safetensors_io import SafetensorsFile, save_file


def load_checkpoint(path: str, device: str = "cpu", keys: Optional[Iterable[str]] = None) -> Dict[str, torch.Tensor]:
    if os.path.isdir(path):
        return load_sharded_checkpoint(path, device, keys)
    want = set(keys) if keys is not None else None
    with SafetensorsFile(path) as sf:
        return {k: sf.get_tensor(k).to(device) for k in sf.keys() if want is None or k in want}


def load_sharded_checkpoint(directory: str, device: str = "cpu", keys: Optional[Iterable[str]] = None) -> Dict[str, torch.Tensor]:
    idx = os.path.join(directory, "model.safetensors.index.json")
    want = set(keys) if keys is not None else None
    out: Dict[str, torch.Tensor] = {}
    if os.path.exists(idx):
        with open(idx) as f:
            wm = json.load(f)["weight_map"]
        by_file: Dict[str, List[str]] = {}
        for k, fn in wm.items():
            if want is None or k in want:
                by_file.setdefault(fn, []).append(k)
        for fn, ks in by_file.items():
            with SafetensorsFile(os.path.join(directory, fn)) as sf:
                for k in ks:
                    out[k] = sf.get_tensor(k).to(device)
        return out
    for fn in sorted(os.listdir(directory)):
        if fn.endswith(".safetensors"):
            out.update(load_checkpoint(os.path.join(directory, fn), device, keys))
    return out


class LazyCheckpoint:
    """Dictionary-like view that reads a tensor from disk only when it is accessed."""

    def __init__(self, path: str):
        self._where: Dict[str, str] = {}
        files = [path] if os.path.isfile(path) else [os.path.join(path, f) for f in sorted(os.listdir(path)) if f.endswith(".safetensors")]
        for fp in files:
            with SafetensorsFile(fp) as sf:
                for k in sf.keys():
                    self._where[k] = fp
        self.reads = 0

    def keys(self):
        return self._where.keys()

    def __contains__(self, k) -> bool:
        return k in self._where

    def __len__(self) -> int:
        return len(self._where)

    def __getitem__(self, k: str) -> torch.Tensor:
        self.reads += 1
        with SafetensorsFile(self._where[k]) as sf:
            return sf.get_tensor(k)


def save_checkpoint(tensors: Dict[str, torch.Tensor], path: str, shard_bytes: Optional[int] = None, metadata: Optional[dict] = None) -> List[str]:
    if shard_bytes is None:
        save_file(tensors, path, metadata=metadata or {"format": "pt"})
        return [path]
    os.makedirs(path, exist_ok=True)
    files, wm, shard, size = [], {}, {}, 0

    def flush():
        nonlocal shard, size
        if shard:
            fn = f"model-{len(files) + 1:05d}.safetensors"
            save_file(shard, os.path.join(path, fn), metadata=metadata or {"format": "pt"})
            wm.update({k: fn for k in shard})
            files.append(fn)
            shard, size = {}, 0

    for k, v in tensors.items():
        shard[k] = v
        size += v.numel() * v.element_size()
        if size >= shard_bytes:
            flush()
    flush()
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": wm}, f)
    return files


def remap_weight_keys(tensors: Dict[str, torch.Tensor], rules: Dict[str, str]) -> Dict[str, torch.Tensor]:
    """``rules``: regex -> replacement, applied in order to every key."""
    out = {}
    for k, v in tensors.items():
        nk = k
        for pat, rep in rules.items():
            nk = re.sub(pat, rep, nk)
        out[nk] = v
    return out


def filter_weights(tensors: Dict[str, torch.Tensor], include: Optional[str] = None, exclude: Optional[str] = None) -> Dict[str, torch.Tensor]:
    return {k: v for k, v in tensors.items() if (include is None or re.search(include, k)) and not (exclude and re.search(exclude, k))}
