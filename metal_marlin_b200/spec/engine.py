"""Speculative decoding loop: draft ``k`` tokens, verify them with one target pass over ``k + 1``
positions, keep the accepted prefix plus one corrected/bonus token, roll the cache back.

Parity: reference ``metal_marlin/speculative/engine.py:153`` (``SpeculativeEngine.generate_step`` ``:387``,
``generate`` ``:496``, adaptive ``num_spec`` ``:667``), ``metal_marlin/inference/mmfp4_pipeline.py:979``
(``_speculative_generate``: one host sync per step, KV truncate ``:1213``) and
``metal_marlin/speculative/verify.py:188`` (tree verification).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..models.transformer import BatchMeta
from .adaptive import AdaptiveSpeculationController, TokenAcceptanceTracker
from .draft import DraftModel, DraftOutput, EagleDraft, MTPDraft, NGramDraft, SmallModelDraft
from .verify import tree_attention_mask, verify_greedy, verify_speculative, verify_tree_greedy


@dataclass
class GenerationStats:
    steps: int = 0
    proposed: int = 0
    accepted: int = 0
    tokens: int = 0
    target_forwards: int = 0

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / max(1, self.proposed)

    @property
    def tokens_per_step(self) -> float:
        return self.tokens / max(1, self.steps)


def make_draft(kind, target_lm, **kw) -> DraftModel:
    if isinstance(kind, DraftModel):
        return kind
    if kind == "ngram":
        return NGramDraft(**kw)
    if kind == "mtp":
        return MTPDraft(target_lm.model, **kw)
    if kind == "eagle":
        return EagleDraft(target_lm.model, **kw)
    if isinstance(kind, str):
        from ..models.mmfp4_causal_lm import MMFP4ForCausalLM
        return SmallModelDraft(MMFP4ForCausalLM.from_pretrained(kind, str(target_lm.device)), **kw)
    return SmallModelDraft(kind, **kw)        # an MMFP4ForCausalLM instance


class SpeculativeEngine:
    def __init__(self, target_lm, draft: DraftModel, num_speculative_tokens: int = 4, adaptive: bool = True,
                 max_len: int = 8192, block_size: int = 16):
        self.lm, self.model, self.draft = target_lm, target_lm.model, draft
        self.k0 = num_speculative_tokens
        self.ctrl = AdaptiveSpeculationController(depth=num_speculative_tokens) if adaptive else None
        self.tracker = TokenAcceptanceTracker()
        self.block_size = block_size
        self.nb = -(-max_len // block_size)
        self.kv = target_lm.new_cache(self.nb, block_size)
        self.bt = torch.arange(self.nb, dtype=torch.int32, device=self.model.device).view(1, self.nb)

    # ------------------------------------------------------------------ target passes
    @torch.no_grad()
    def _target(self, tokens: Sequence[int], start: int, tree_parents: Optional[List[int]] = None, n_tree: int = 0
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        """Run the target over ``tokens`` placed at cache positions ``start ..``.  Returns (logits [T, V],
        final normalised hidden [T, H]).  With ``tree_parents`` the last ``n_tree`` tokens are tree nodes:
        their rotary position is context length + depth and they attend through a tree mask."""
        dev = self.model.device
        T = len(tokens)
        slots = torch.arange(start, start + T, dtype=torch.int64, device=dev)
        pos = list(range(start, start + T))
        mask = None
        if tree_parents is not None and n_tree:
            base = start + T - n_tree
            depth = []
            for i, p in enumerate(tree_parents):
                depth.append(0 if p < 0 else depth[p] + 1)
            for i in range(n_tree):
                pos[T - n_tree + i] = base + depth[i]
            n_ctx = start + T
            mask = torch.zeros(T, n_ctx, dtype=torch.bool, device=dev)
            q_abs = torch.arange(start, start + T, device=dev).unsqueeze(1)
            k_abs = torch.arange(n_ctx, device=dev).unsqueeze(0)
            mask[:] = k_abs <= q_abs
            mask[:, base:] = False
            mask[T - n_tree:, base:] = tree_attention_mask(tree_parents, dev)
            lin = T - n_tree
            if lin:
                mask[:lin, start:base] = torch.tril(torch.ones(lin, lin, dtype=torch.bool, device=dev))
        meta = BatchMeta(positions=torch.tensor(pos, dtype=torch.int32, device=dev), slots=slots, block_tables=self.bt,
                         ctx_lens=torch.tensor([start + T], dtype=torch.int32, device=dev), decode=False,
                         cu_seqlens=[0, T], ctx_lens_host=[start + T])
        meta.attn_mask = mask
        h, d = self.model.forward_hidden(torch.tensor(list(tokens), dtype=torch.int64, device=dev), self.kv, meta)
        return self.model.logits(h, d), self.model.final_hidden(h, d)

    def _move_kv(self, src_positions: List[int], dst_start: int) -> None:
        """Copy cache rows of accepted tree nodes into consecutive positions."""
        if src_positions == list(range(dst_start, dst_start + len(src_positions))):
            return
        src = torch.tensor(src_positions, device=self.model.device)
        dst = torch.arange(dst_start, dst_start + len(src_positions), device=self.model.device)
        for pool in (self.kv.k, self.kv.v):
            for t in pool:
                if t is not None:
                    ops.kv_copy_rows(t, dst, src)

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, prompt_ids: Sequence[int], max_new_tokens: int = 64, temperature: float = 0.0, seed: int = 0,
                 eos_ids: Sequence[int] = ()) -> Tuple[List[int], GenerationStats]:
        gen = torch.Generator().manual_seed(seed)
        stats = GenerationStats()
        ctx = list(prompt_ids)
        self.draft.reset()
        logits, hidden = self._target(ctx, 0)
        stats.target_forwards += 1
        cached = len(ctx)                       # positions [0, cached) hold valid KV
        nxt = self._pick(logits[-1], temperature, gen)
        out = [nxt]
        last_hidden = hidden[-1]
        while len(out) < max_new_tokens and out[-1] not in eos_ids:
            k = min(self.ctrl.depth if self.ctrl else self.k0, max_new_tokens - len(out))
            prop: DraftOutput = self.draft.propose(ctx + out, k, hidden=last_hidden) if k > 0 else DraftOutput([])
            stats.steps += 1
            if prop.parents is not None and prop.tokens:
                n_acc, new_tokens, last_hidden = self._step_tree(ctx + out, cached, prop)
            else:
                n_acc, new_tokens, last_hidden = self._step_linear(ctx + out, cached, prop, temperature, gen)
            stats.target_forwards += 1
            stats.proposed += len(prop.tokens)
            stats.accepted += n_acc
            self.tracker.record(prop.tokens if prop.parents is None else prop.tokens[:max(n_acc, 1)], n_acc)
            if self.ctrl:
                self.ctrl.update(len(prop.tokens) if prop.parents is None else max(1, len(set(prop.parents))), n_acc)
            cached = len(ctx) + len(out) + n_acc
            for t in new_tokens:
                out.append(t)
                if t in eos_ids or len(out) >= max_new_tokens:
                    break
        stats.tokens = len(out)
        return out[:max_new_tokens], stats

    @staticmethod
    def _pick(logits: torch.Tensor, temperature: float, gen) -> int:
        if temperature <= 0:
            return int(logits.argmax())
        return int(torch.multinomial(torch.softmax(logits.float() / temperature, -1).cpu(), 1, generator=gen))

    def _step_linear(self, seq: List[int], cached: int, prop: DraftOutput, temperature: float, gen):
        """``seq[cached:]`` is the not-yet-cached tail (exactly the last sampled token)."""
        feed = seq[cached:] + prop.tokens
        logits, hidden = self._target(feed, cached)
        n_tail = len(seq) - cached
        rows = logits[n_tail - 1:]                        # row i: distribution for draft i (K + 1 rows)
        if temperature <= 0:
            res = verify_greedy(rows, prop.tokens)
        else:
            res = verify_speculative(torch.softmax(rows.float() / temperature, -1).cpu(),
                                     None if prop.probs is None else prop.probs.cpu(), prop.tokens, gen)
        n = res.num_accepted
        return n, prop.tokens[:n] + [res.next_token], hidden[n_tail - 1 + n]

    def _step_tree(self, seq: List[int], cached: int, prop: DraftOutput):
        tail = seq[cached:]
        feed = tail + prop.tokens
        logits, hidden = self._target(feed, cached, tree_parents=prop.parents, n_tree=len(prop.tokens))
        n_tail = len(tail)
        path, nxt = verify_tree_greedy(logits[n_tail - 1], logits[n_tail:], prop.tokens, prop.parents)
        base = cached + n_tail
        self._move_kv([base + i for i in path], base)
        toks = [prop.tokens[i] for i in path]
        last = hidden[n_tail + path[-1]] if path else hidden[n_tail - 1]
        return len(path), toks + [nxt], last
