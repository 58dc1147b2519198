"""Draft token sources for speculative decoding.

Parity: reference ``metal_marlin/speculative/draft.py``: ``DraftModel`` ABC ``:64``, ``SmallModelDraft``
``:102``, ``NGramDraft`` ``:272`` (online n-gram table), ``EagleHead`` ``:459/:550`` (tree drafts);
``metal_marlin/speculative/mtp_draft.py:17`` / ``metal_marlin/layers/mmfp4_mtp_head.py:39`` (multi-token
prediction heads sharing the target's lm_head).
"""
from __future__ import annotations

import abc
from collections import defaultdict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch


@dataclass
class DraftOutput:
    tokens: List[int]
    probs: Optional[torch.Tensor] = None          # [K, V] draft distributions (None = deterministic draft)
    parents: Optional[List[int]] = None           # tree drafts: parent index of every node (-1 = context)


class DraftModel(abc.ABC):
    @abc.abstractmethod
    def propose(self, context: Sequence[int], k: int, hidden: Optional[torch.Tensor] = None) -> DraftOutput:
        ...

    def observe(self, context: Sequence[int]) -> None:
        """Feed accepted tokens back (online drafts learn from them)."""

    def reset(self) -> None:
        pass


class NGramDraft(DraftModel):
    """Prompt-lookup / online n-gram table: the longest suffix seen before predicts what followed it."""

    def __init__(self, max_n: int = 4, min_n: int = 1):
        self.max_n, self.min_n = max_n, min_n
        self.table: Dict[Tuple[int, ...], Dict[int, int]] = defaultdict(lambda: defaultdict(int))
        self._seen = 0

    def reset(self) -> None:
        self.table.clear()
        self._seen = 0

    def observe(self, context: Sequence[int]) -> None:
        ctx = list(context)
        for i in range(max(self._seen, 1), len(ctx)):
            for n in range(self.min_n, self.max_n + 1):
                if i - n < 0:
                    break
                self.table[tuple(ctx[i - n:i])][ctx[i]] += 1
        self._seen = len(ctx)

    def _next(self, ctx: List[int]) -> Optional[int]:
        for n in range(min(self.max_n, len(ctx)), self.min_n - 1, -1):
            nxt = self.table.get(tuple(ctx[-n:]))
            if nxt:
                return max(nxt.items(), key=lambda kv: (kv[1], -kv[0]))[0]
        return None

    def propose(self, context, k, hidden=None) -> DraftOutput:
        self.observe(context)
        ctx, out = list(context), []
        for _ in range(k):
            t = self._next(ctx)
            if t is None:
                break
            out.append(t)
            ctx.append(t)
        return DraftOutput(out)


class SmallModelDraft(DraftModel):
    """A smaller causal LM with the target's vocabulary drafts ``k`` tokens autoregressively.  It keeps
    its own paged cache and only prefills the tokens it has not seen yet."""

    def __init__(self, lm, max_len: int = 8192, block_size: int = 16, temperature: float = 0.0):
        from ..models.mmfp4_causal_lm import prefill
        self.lm, self._prefill = lm, prefill
        self.block_size = block_size
        self.nb = -(-max_len // block_size)
        self.kv = lm.new_cache(self.nb, block_size)
        self.bt = torch.arange(self.nb, dtype=torch.int32).view(1, self.nb)
        self.cached: List[int] = []
        self.temperature = temperature

    def reset(self) -> None:
        self.cached = []

    @torch.no_grad()
    def propose(self, context, k, hidden=None) -> DraftOutput:
        ctx = list(context)
        common = 0
        for a, b in zip(self.cached, ctx):
            if a != b:
                break
            common += 1
        common = min(common, len(ctx) - 1)
        toks, probs = [], []
        cur = ctx
        for _ in range(k):
            lg = self._prefill(self.lm.model, self.kv, [cur], self.bt, start=[common])[0]
            if self.temperature > 0:
                p = torch.softmax(lg / self.temperature, -1)
                t = int(torch.multinomial(p.cpu(), 1))
                probs.append(p)
            else:
                t = int(lg.argmax())
            common = len(cur)
            toks.append(t)
            cur = cur + [t]
        self.cached = cur[:-1]
        return DraftOutput(toks, torch.stack(probs) if probs else None)


class MTPHead:
    """Multi-token-prediction module: depth ``d`` maps the target's final hidden state (plus the embedding
    of the last drafted token) to a hidden state whose head projection predicts token ``t + d + 1``.
    Weights: per depth one ``[H, 2H]`` bf16 projection; the target's final norm and lm_head are shared."""

    def __init__(self, model, depth: int = 4, seed: int = 0, std: float = 0.02):
        H = model.cfg.hidden_size
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.model, self.depth = model, depth
        self.proj = [(torch.randn(H, 2 * H, generator=g) * std).to(torch.bfloat16).to(model.device) for _ in range(depth)]

    @torch.no_grad()
    def draft(self, hidden: torch.Tensor, last_token: int, k: int) -> List[int]:
        m = self.model
        h = hidden.reshape(1, -1).to(torch.bfloat16)
        tok = last_token
        out = []
        for d in range(min(k, self.depth)):
            e = m.embed[tok].reshape(1, -1)
            h = torch.nn.functional.linear(torch.cat([h, e], -1).float(), self.proj[d].float()).to(torch.bfloat16)
            lg = torch.nn.functional.linear(h.float(), m.lm_head.float())
            tok = int(lg.argmax(-1))
            out.append(tok)
        return out


class MTPDraft(DraftModel):
    def __init__(self, model, depth: int = 4, seed: int = 0):
        if model.mtp is None:
            model.mtp = MTPHead(model, depth, seed)
        self.head = model.mtp

    def propose(self, context, k, hidden=None) -> DraftOutput:
        if hidden is None:
            return DraftOutput([])
        return DraftOutput(self.head.draft(hidden, context[-1], k))


class EagleDraft(DraftModel):
    """EAGLE-style tree draft: a light autoregressive head expands the ``width`` most likely continuations
    per level for ``depth`` levels; the tree is verified in one target pass with a tree attention mask."""

    def __init__(self, model, width: int = 3, depth: int = 3, seed: int = 0):
        self.model, self.width, self.depth = model, width, depth
        self.head = MTPHead(model, depth, seed + 17)

    @torch.no_grad()
    def propose(self, context, k, hidden=None) -> DraftOutput:
        if hidden is None:
            return DraftOutput([], parents=[])
        m = self.model
        tokens, parents = [], []
        frontier = [(-1, hidden.reshape(1, -1).to(torch.bfloat16), context[-1])]
        for d in range(self.depth):
            nxt = []
            for parent, h, tok in frontier:
                e = m.embed[tok].reshape(1, -1)
                hh = torch.nn.functional.linear(torch.cat([h, e], -1).float(), self.head.proj[d].float()).to(torch.bfloat16)
                lg = torch.nn.functional.linear(hh.float(), m.lm_head.float())[0]
                top = lg.topk(self.width if d == 0 else 1).indices.tolist()
                for t in top:
                    tokens.append(t)
                    parents.append(parent)
                    nxt.append((len(tokens) - 1, hh, t))
            frontier = nxt
            if len(tokens) >= max(k, 1) * self.width:
                break
        return DraftOutput(tokens, parents=parents)
