"""Weights & Biases logging that degrades to a local JSON-lines file when the ``wandb`` package (or a network) is
missing: the same ``init / log / finish`` calls work everywhere, benchmark and quantization drivers log through it.

Parity: reference ``metal_marlin/wandb_helper.py:22-70`` (``WandbHelper.init``, ``log``, ``finish``, module-level helper).
"""
from __future__ import annotations

import json
import os
import time
from typing import Any, Dict, List, Optional


class WandbHelper:
    def __init__(self, fallback_dir: Optional[str] = None) -> None:
        self._run = None
        self._wandb = None
        self._file = None
        self._step = 0
        self.fallback_dir = fallback_dir or os.environ.get("METAL_MARLIN_LOG_DIR", ".")
        self.enabled = os.environ.get("WANDB_MODE", "") != "disabled"

    @property
    def backend(self) -> str:
        return "wandb" if self._run is not None else ("jsonl" if self._file is not None else "none")

    def init(self, project: Optional[str] = None, name: Optional[str] = None, config: Optional[Dict[str, Any]] = None,
             tags: Optional[List[str]] = None, **kwargs: Any) -> Any:
        if self.enabled:
            try:
                import wandb  # type: ignore
                self._wandb = wandb
                self._run = wandb.init(project=project, name=name, config=config, tags=tags, **kwargs)
                return self._run
            except Exception:
                self._run = None
        os.makedirs(self.fallback_dir, exist_ok=True)
        path = os.path.join(self.fallback_dir, f"{project or 'run'}-{name or time.strftime('%Y%m%d-%H%M%S')}.jsonl")
        self._file = open(path, "a")
        self._file.write(json.dumps({"_event": "init", "project": project, "name": name, "config": config or {}, "tags": tags or []}) + "\n")
        self.path = path
        return None

    def log(self, data: Dict[str, Any], step: Optional[int] = None, **kwargs: Any) -> None:
        self._step = self._step + 1 if step is None else int(step)
        if self._run is not None:
            self._wandb.log(data, step=self._step, **kwargs)
        elif self._file is not None:
            self._file.write(json.dumps({"_step": self._step, "_time": time.time(), **{k: _plain(v) for k, v in data.items()}}) + "\n")
            self._file.flush()

    def finish(self) -> None:
        if self._run is not None:
            self._run.finish()
            self._run = None
        if self._file is not None:
            self._file.write(json.dumps({"_event": "finish", "steps": self._step}) + "\n")
            self._file.close()
            self._file = None


def _plain(v: Any) -> Any:
    try:
        import torch
        if isinstance(v, torch.Tensor):
            return v.item() if v.numel() == 1 else v.tolist()
    except Exception:
        pass
    if isinstance(v, (int, float, str, bool)) or v is None:
        return v
    if isinstance(v, (list, tuple)):
        return [_plain(x) for x in v]
    if isinstance(v, dict):
        return {str(k): _plain(x) for k, x in v.items()}
    return str(v)


_default: Optional[WandbHelper] = None


def get_wandb() -> WandbHelper:
    global _default
    if _default is None:
        _default = WandbHelper()
    return _default
