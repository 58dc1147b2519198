"""Early-exit decoding: run the decoder layer by layer and stop as soon as the head is confident.

After every ``check_every`` layers (from ``min_layers`` on) the running hidden state goes through the final norm and the
LM head; when the largest soft-max probability of every sequence reaches ``exit_threshold`` the remaining layers are
skipped for this token.  The KV rows of the skipped layers are not written, so a later token that runs deeper attends to
fewer keys there - the usual early-exit approximation.

Works on the shared :class:`~metal_marlin_b200.models.transformer.Transformer` (MLA or GQA, dense or MoE).

Parity: reference ``metal_marlin/early_exit.py:21-160`` (``EarlyExitOutput``, ``EarlyExitModel.forward`` with
``exit_threshold``, ``exit_layer``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..models.transformer import BatchMeta, PagedKVStorage, Transformer


@dataclass
class EarlyExitOutput:
    logits: torch.Tensor            # fp32 [rows, vocab]
    exit_layer: int                 # index of the last layer that ran (num_layers - 1 = no early exit)
    confidence: torch.Tensor        # [rows] max soft-max probability at the exit


class EarlyExitModel:
    def __init__(self, model: Transformer, exit_threshold: float = 0.9, min_layers: int = 1, check_every: int = 1):
        self.model, self.exit_threshold, self.min_layers, self.check_every = model, float(exit_threshold), int(min_layers), max(1, int(check_every))
        self.exit_counts = [0] * len(model.layers)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, kv: PagedKVStorage, meta: BatchMeta, rows: Optional[torch.Tensor] = None) -> EarlyExitOutput:
        m = self.model
        if m.tp is not None:
            m.tp.begin_step()
        h = ops.embedding(m.embed, input_ids)
        d = None
        n = len(m.layers)
        logits = conf = None
        exit_layer = n - 1
        for li, L in enumerate(m.layers):
            h, d = (m._attn_mla if m.cfg.is_mla else m._attn_gqa)(L, li, h, d, kv, meta)
            h, d = (m._mlp_moe if L.router_w is not None else m._mlp_dense)(L, li, h, d)
            last = li == n - 1
            if last or (li + 1 >= self.min_layers and (li + 1 - self.min_layers) % self.check_every == 0):
                dd = m.tp.finish_plain(d) if getattr(d, "pending_rs", False) else d
                logits = m.logits(h, dd, rows)
                if m.tp is not None and m.tp.tp > 1:
                    logits = m.full_logits(logits)
                conf = torch.softmax(logits.float(), -1).amax(-1)
                d = dd
                if last or bool((conf >= self.exit_threshold).all()):
                    exit_layer = li
                    break
        self.exit_counts[exit_layer] += 1
        return EarlyExitOutput(logits=logits, exit_layer=exit_layer, confidence=conf)

    __call__ = forward

    def average_exit_layer(self) -> float:
        tot = sum(self.exit_counts)
        return sum(i * c for i, c in enumerate(self.exit_counts)) / tot if tot else float(len(self.exit_counts) - 1)
