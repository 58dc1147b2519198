"""Pipeline parallelism: consecutive layer ranges on consecutive ranks, activations handed over point to point.

Parity: reference ``metal_marlin/distributed/pipeline_parallel.py`` (stage assignment, micro-batch schedule).  Each
stage is a ``Transformer`` holding only its layers (the first stage also the embedding, the last the final norm and
the head); the hand-over is the (hidden, pending delta) pair of the residual stream.  Prefill runs a fill-drain
schedule over micro-batches; decode, one token per step, is inherently sequential across stages and is meant for
models that do not fit a tensor-parallel group.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..models.transformer import BatchMeta, PagedKVStorage, Transformer


def stage_layers(n_layers: int, pp: int) -> List[Tuple[int, int]]:
    """Contiguous, balanced layer ranges (earlier stages take the remainder)."""
    base, rem = divmod(n_layers, pp)
    out, s = [], 0
    for p in range(pp):
        n = base + (1 if p < rem else 0)
        out.append((s, s + n))
        s += n
    return out


class PipelineStage:
    def __init__(self, model: Transformer, stage: int, pp: int, prev_rank: Optional[int], next_rank: Optional[int], group=None):
        self.cfg = model.cfg
        self.stage, self.pp, self.prev, self.next, self.group = stage, pp, prev_rank, next_rank, group
        lo, hi = stage_layers(len(model.layers), pp)[stage]
        self.lo, self.hi = lo, hi
        self.model = model
        self.layers = model.layers[lo:hi]
        self.is_first, self.is_last = stage == 0, stage == pp - 1

    def _run_layers(self, h, d, kv: PagedKVStorage, meta: BatchMeta):
        m = self.model
        for off, L in enumerate(self.layers):
            li = self.lo + off
            h, d = (m._attn_mla if self.cfg.is_mla else m._attn_gqa)(L, li, h, d, kv, meta)
            h, d = (m._mlp_moe if L.router_w is not None else m._mlp_dense)(L, li, h, d)
        return h, d

    def _recv(self, T: int, device):
        buf = torch.empty(2, T, self.cfg.hidden_size, dtype=torch.bfloat16, device=device)
        dist.recv(buf, src=self.prev, group=self.group)
        return buf[0], buf[1]

    def _send(self, h, d):
        buf = torch.stack([h, d if d is not None else torch.zeros_like(h)]).contiguous()
        dist.send(buf, dst=self.next, group=self.group)

    def forward(self, input_ids: torch.Tensor, kv: PagedKVStorage, meta: BatchMeta, rows: Optional[torch.Tensor] = None):
        """One micro-batch through this stage.  The last stage returns fp32 logits of ``rows``, others ``None``."""
        if self.is_first:
            h, d = ops.embedding(self.model.embed, input_ids), None
        else:
            h, d = self._recv(input_ids.numel(), self.model.device)
        h, d = self._run_layers(h, d, kv, meta)
        if self.is_last:
            return self.model.logits(h, d, rows)
        self._send(h, d)
        return None


def pipeline_prefill(stage: PipelineStage, microbatches: Sequence[Tuple[torch.Tensor, PagedKVStorage, BatchMeta, Optional[torch.Tensor]]]):
    """Fill-drain schedule: with blocking hand-overs every stage simply processes the micro-batches in order; stage s
    works on micro-batch i while stage s + 1 works on i - 1.  Returns the list of logits on the last stage."""
    outs = []
    for ids, kv, meta, rows in microbatches:
        o = stage.forward(ids, kv, meta, rows)
        if o is not None:
            outs.append(o)
    return outs
