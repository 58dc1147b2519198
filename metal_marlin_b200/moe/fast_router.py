"""Batch router with a cache of hot expert pairs: gate product, top-k choice and weights for a batch of tokens in one call,
plus bookkeeping of which (first, second) expert pairs keep recurring — the pairs a prefetcher or a fused two-expert path
wants to know about.

Activations may arrive as a bf16 tensor or as their raw 16-bit patterns (a ``uint16`` array, the layout the reference passes
across its C++ boundary); the gate runs through ``ops.moe_router`` (the router kernel on a GPU).

Parity: reference ``moe_router_cpp.py:50`` (``MoERouterCpp``: ``route_batch``, ``hot_pair_count``, ``reset_hot_pair_cache``, properties).
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch


def is_available() -> bool:
    return True


@dataclass
class RouterBatchOutput:
    expert_ids: torch.Tensor             # int32 [tokens, top_k]
    expert_weights: torch.Tensor         # fp32 [tokens, top_k], renormalised
    num_tokens: int
    hot_pair_hits: int                   # tokens of this batch whose leading pair was in the cache already
    hot_pairs: List[Tuple[int, int]]     # current cache content, most recently used last

    @property
    def top_k(self) -> int:
        return int(self.expert_ids.shape[1])


class MoERouterCpp:
    def __init__(self, num_experts: int, hidden_dim: int, top_k: int, max_batch_tokens: int = 128, hot_pair_cache_capacity: int = 256,
                 hot_pair_threshold: int = 8, scoring: int = 0, renorm: bool = True, device=None):
        if top_k > num_experts:
            raise ValueError(f"top_k {top_k} exceeds the number of experts {num_experts}")
        self._E, self._H, self._K = num_experts, hidden_dim, top_k
        self.max_batch_tokens = max_batch_tokens
        self.capacity, self.threshold = hot_pair_cache_capacity, hot_pair_threshold
        self.scoring, self.renorm = scoring, renorm
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self._pair_counts: Dict[Tuple[int, int], int] = {}
        self._hot: "OrderedDict[Tuple[int, int], int]" = OrderedDict()
        self._w_key, self._w_dev = None, None

    num_experts = property(lambda self: self._E)
    hidden_dim = property(lambda self: self._H)
    top_k = property(lambda self: self._K)

    @property
    def hot_pair_count(self) -> int:
        return len(self._hot)

    def reset_hot_pair_cache(self) -> None:
        self._pair_counts.clear()
        self._hot.clear()

    def _activations(self, a) -> torch.Tensor:
        if isinstance(a, np.ndarray):
            if a.dtype != np.uint16:
                raise TypeError(f"array activations must be uint16 bit patterns of bfloat16, got {a.dtype}")
            a = torch.from_numpy(a.astype(np.int16)).view(torch.bfloat16)
        if a.dim() != 2 or a.shape[1] != self._H:
            raise ValueError(f"activations must be [tokens, {self._H}], got {tuple(a.shape)}")
        if a.shape[0] > self.max_batch_tokens:
            raise ValueError(f"{a.shape[0]} tokens exceed max_batch_tokens = {self.max_batch_tokens}")
        return a.to(self.device, torch.bfloat16 if self.device.type == "cuda" else torch.float32)

    def _weights(self, w) -> torch.Tensor:
        key = (id(w), getattr(w, "data_ptr", lambda: 0)() if isinstance(w, torch.Tensor) else w.__array_interface__["data"][0])
        if key != self._w_key:
            t = torch.as_tensor(np.ascontiguousarray(w, dtype=np.float32)) if isinstance(w, np.ndarray) else w
            if tuple(t.shape) != (self._E, self._H):
                raise ValueError(f"router weights must be [{self._E}, {self._H}], got {tuple(t.shape)}")
            self._w_dev = t.to(self.device, torch.bfloat16 if self.device.type == "cuda" else torch.float32).contiguous()
            self._w_key = key
        return self._w_dev

    def route_batch(self, token_activations, router_weights, router_bias=None) -> RouterBatchOutput:
        from .. import ops
        x, w = self._activations(token_activations), self._weights(router_weights)
        bias = None
        if router_bias is not None:
            bias = torch.as_tensor(np.asarray(router_bias, dtype=np.float32) if isinstance(router_bias, np.ndarray) else router_bias).to(self.device, torch.float32)
        if bias is not None and self.scoring == 0:
            # soft-max gates take the bias inside the logits; the router op's bias argument is the selection-only correction of sigmoid gates
            logits = x.float() @ w.float().t() + bias
            p = torch.softmax(logits, -1)
            wt, ids = p.topk(self._K, -1)
            wt = wt / wt.sum(-1, keepdim=True) if self.renorm else wt
            ids = ids.to(torch.int32)
        else:
            ids, wt = ops.moe_router(x, w, bias=bias, topk=self._K, scoring=self.scoring, renorm=self.renorm)
        ids_c = ids.cpu()
        hits = 0
        if self._K >= 2:
            for a, b in ids_c[:, :2].tolist():
                pair = (a, b) if a < b else (b, a)
                if pair in self._hot:
                    hits += 1
                    self._hot.move_to_end(pair)
                    self._hot[pair] += 1
                    continue
                n = self._pair_counts.get(pair, 0) + 1
                if n >= self.threshold:
                    self._pair_counts.pop(pair, None)
                    self._hot[pair] = n
                    while len(self._hot) > self.capacity:
                        self._hot.popitem(last=False)
                else:
                    self._pair_counts[pair] = n
        return RouterBatchOutput(ids_c.to(torch.int32), wt.float().cpu(), int(x.shape[0]), hits, list(self._hot))
