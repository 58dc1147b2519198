"""``TrellisGenerator``: text generation over a ``TrellisForCausalLM`` (sampling, repetition penalty, streaming).

Parity: reference ``metal_marlin/trellis/generate.py:41`` (``GenerationConfig``), ``:68`` (``TrellisGenerator.generate`` /
``stream_generate``) and the sampling rules of ``metal_marlin/trellis/lm.py:569-641``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterator, List, Optional, Sequence, Union

import torch

from ..engine.session import DecodeSession, SamplingParams
from ..models.mmfp4_causal_lm import prefill


@dataclass
class GenerationConfig:
    max_new_tokens: int = 128
    temperature: float = 0.7
    top_k: int = 50
    top_p: float = 0.9
    repetition_penalty: float = 1.1
    do_sample: bool = True
    eos_token_id: Optional[Union[int, Sequence[int]]] = None
    seed: int = 0


class TrellisGenerator:
    def __init__(self, model, tokenizer=None):
        self.model, self.tokenizer = model, tokenizer

    def _ids(self, prompt) -> List[int]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a tokenizer is needed for text prompts")
            return list(self.tokenizer.encode(prompt))
        return [int(t) for t in prompt]

    def _sampling(self, cfg: GenerationConfig) -> SamplingParams:
        greedy = (not cfg.do_sample) or cfg.temperature == 0
        return SamplingParams(temperature=0.0 if greedy else cfg.temperature, top_k=cfg.top_k, top_p=cfg.top_p,
                              repetition_penalty=cfg.repetition_penalty, seed=cfg.seed)

    def stream_generate(self, prompt, config: Optional[GenerationConfig] = None) -> Iterator[int]:
        """Yield new token ids one at a time."""
        cfg = config or GenerationConfig()
        ids = self._ids(prompt)
        lm = self.model
        bs = 16
        nb = (len(ids) + cfg.max_new_tokens + bs) // bs
        kv = lm.new_cache(nb, bs)
        bt = torch.arange(nb, dtype=torch.int32).view(1, nb)
        logits = prefill(lm.model, kv, [ids], bt)
        sess = DecodeSession(lm.model, kv, 1, nb, max_new_tokens=cfg.max_new_tokens, use_graph=False)
        sess.set_sampling([self._sampling(cfg)])
        first = sess.sample_first(logits, history=[ids]) if hasattr(sess, "sample_first") else logits.argmax(-1)
        sess.set_state(first, [len(ids)], bt)
        eos = cfg.eos_token_id
        eos = set([eos] if isinstance(eos, int) else (eos or []))
        tok = int(first[0])
        yield tok
        for _ in range(cfg.max_new_tokens - 1):
            if tok in eos:
                return
            tok = int(sess.step()[0])
            yield tok

    def generate(self, prompt, config: Optional[GenerationConfig] = None):
        out = list(self.stream_generate(prompt, config))
        if isinstance(prompt, str) and self.tokenizer is not None:
            return self.tokenizer.decode(out)
        return out
