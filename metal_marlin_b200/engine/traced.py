"""A decoder layer captured once into a CUDA graph at a fixed ``[batch, seq, hidden]`` shape and replayed: one launch for
the layer's whole kernel sequence instead of one per operator.

The layer is any callable ``layer(hidden_states, **static_kwargs) -> tensor | tuple`` whose other inputs do not change between
calls (or are tensors updated in place, e.g. a position tensor): they are bound at ``compile``.  Input is copied into a static
buffer, the graph is replayed, the static output is returned (valid until the next call; ``clone`` it to keep it).  On a CPU
the layer simply runs.

Parity: reference ``traced/mpsgraph_layer.py:17`` (``TracedDecoderLayer``: whole-layer graph compilation).
"""
from __future__ import annotations

from typing import Any, Callable, Optional

import torch


class TracedDecoderLayer:
    def __init__(self, layer: Callable, batch_size: int = 1, seq_len: int = 1, hidden_size: int = 2048, dtype: torch.dtype = torch.bfloat16,
                 device=None, warmup: int = 2):
        self.layer = layer
        self.batch_size, self.seq_len, self.hidden_size = batch_size, seq_len, hidden_size
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.dtype, self.warmup = dtype, warmup
        self._graph: Optional[Any] = None
        self._in: Optional[torch.Tensor] = None
        self._out: Any = None
        self._kwargs: dict = {}
        self._compiled = False
        self.replays = 0

    @property
    def shape(self):
        return (self.batch_size, self.seq_len, self.hidden_size)

    @staticmethod
    def _first(out):
        return out[0] if isinstance(out, (tuple, list)) else out

    def compile(self, **static_kwargs) -> "TracedDecoderLayer":
        if self._compiled:
            return self
        self._kwargs = static_kwargs
        self._in = torch.zeros(self.shape, dtype=self.dtype, device=self.device)
        if self.device.type == "cuda":
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side), torch.no_grad():
                for _ in range(self.warmup):
                    self.layer(self._in, **static_kwargs)
            torch.cuda.current_stream(self.device).wait_stream(side)
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph), torch.no_grad():
                self._out = self._first(self.layer(self._in, **static_kwargs))
        self._compiled = True
        return self

    def __call__(self, hidden_states: torch.Tensor, **kwargs) -> torch.Tensor:
        if tuple(hidden_states.shape) != self.shape:
            raise ValueError(f"traced for {self.shape}, got {tuple(hidden_states.shape)}")
        if not self._compiled:
            self.compile(**kwargs)
        elif kwargs and any(kwargs.get(k) is not v for k, v in self._kwargs.items()):
            raise ValueError("the layer was captured with other keyword arguments; update tensors in place or build a new traced layer")
        if self._graph is None:
            with torch.no_grad():
                return self._first(self.layer(hidden_states.to(self.dtype), **self._kwargs))
        self._in.copy_(hidden_states)
        self._graph.replay()
        self.replays += 1
        return self._out
