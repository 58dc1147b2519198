"""Token samplers: ``SamplingConfig`` + ``Sampler`` (argmax, temperature, top-k, top-p, min-p, repetition
penalty) and ``sample_next_token``.

Parity: reference ``metal_marlin/sampler.py:57-537`` (``SamplingConfig``, ``MetalSampler.sample``,
``sample_next_token``) and the filter order of ``metal_marlin/inference/mmfp4_pipeline.py:224-425``:
repetition penalty -> temperature -> top-k -> top-p -> min-p -> categorical draw.  On CUDA tensors every call
is one launch of the fused sampling kernel (``csrc/sampling.cu``); on CPU the PyTorch restatement runs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from . import ops


@dataclass
class SamplingConfig:
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    seed: Optional[int] = None
    do_sample: bool = True

    def validate(self) -> "SamplingConfig":
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not 0.0 <= self.min_p < 1.0:
            raise ValueError("min_p must be in [0, 1)")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be > 0")
        return self

    @property
    def greedy(self) -> bool:
        return (not self.do_sample) or self.temperature == 0.0


class Sampler:
    """Stateful sampler for a batch: keeps the per-row parameter tensors on the device and a draw counter so
    successive calls use fresh random numbers (counter-based Philox in the kernel)."""

    def __init__(self, vocab_size: int, device=None):
        self.vocab_size = vocab_size
        self.device = torch.device(device) if device is not None else None
        self._draws = 0

    def _vec(self, vals: Sequence[float], dtype, device):
        return torch.tensor(list(vals), dtype=dtype, device=device)

    def sample(self, logits: torch.Tensor, configs, history: Optional[torch.Tensor] = None,
               return_logprob: bool = False):
        """``logits [B, V]`` fp32; ``configs`` one ``SamplingConfig`` or a list per row; ``history [B, L]`` int64
        (negative = padding) feeds the repetition penalty."""
        if logits.dim() == 1:
            logits = logits.unsqueeze(0)
        B = logits.shape[0]
        cfgs: List[SamplingConfig] = [configs] * B if isinstance(configs, SamplingConfig) else list(configs)
        dev = logits.device
        logits = logits.to(torch.float32)
        if all(c.greedy and c.repetition_penalty == 1.0 for c in cfgs):
            ids = ops.argmax(logits)
            if return_logprob:
                lp = torch.log_softmax(logits, -1).gather(1, ids.view(-1, 1)).squeeze(1)
                return ids, lp
            return ids
        seed = next((c.seed for c in cfgs if c.seed is not None), 0)
        self._draws += 1
        lp = torch.empty(B, dtype=torch.float32, device=dev)
        gen = None
        if not logits.is_cuda:
            gen = torch.Generator().manual_seed(int(seed) * 1000003 + self._draws)
        ids = ops.sample(
            logits, temperature=self._vec([0.0 if c.greedy else c.temperature for c in cfgs], torch.float32, dev),
            top_k=self._vec([c.top_k for c in cfgs], torch.int32, dev), top_p=self._vec([c.top_p for c in cfgs], torch.float32, dev),
            min_p=self._vec([c.min_p for c in cfgs], torch.float32, dev), history=history,
            rep_penalty=self._vec([c.repetition_penalty for c in cfgs], torch.float32, dev) if history is not None else None,
            seed=seed, offset=self._draws, out_logprob=lp, generator=gen)
        return (ids, lp) if return_logprob else ids

    # reference-compatible conveniences
    def argmax(self, logits: torch.Tensor) -> torch.Tensor:
        return ops.argmax(logits.to(torch.float32) if logits.dim() == 2 else logits.to(torch.float32).unsqueeze(0))

    def sample_top_k(self, logits, k: int, temperature: float = 1.0):
        return self.sample(logits, SamplingConfig(temperature=temperature, top_k=k))

    def sample_top_p(self, logits, p: float, temperature: float = 1.0):
        return self.sample(logits, SamplingConfig(temperature=temperature, top_p=p))

    def sample_categorical(self, logits, temperature: float = 1.0):
        return self.sample(logits, SamplingConfig(temperature=temperature))


def sample_next_token(logits: torch.Tensor, config: Optional[SamplingConfig] = None, generated: Optional[Sequence[int]] = None,
                      sampler: Optional[Sampler] = None) -> int:
    """One token id from ``logits [V]`` (or ``[1, V]``)."""
    config = (config or SamplingConfig()).validate()
    sampler = sampler or Sampler(logits.shape[-1], logits.device)
    hist = None
    if generated and config.repetition_penalty != 1.0:
        hist = torch.tensor([list(generated)], dtype=torch.int64, device=logits.device)
    return int(sampler.sample(logits.view(1, -1), config, history=hist)[0])
