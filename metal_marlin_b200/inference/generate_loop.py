"""A generation loop for models with the Hugging Face call convention (``model(input_ids=..., past_key_values=..., use_cache=True)``
returning ``.logits`` and ``.past_key_values``) that allocates once: one output buffer for prompt + new tokens, one-token input
views into it, sampling through this package's sampling kernel.  The engine's own models generate through
``MMFP4Pipeline`` / ``LLMEngine``; this loop serves wrapped ``transformers`` models (for instance after ``hf.replace_linear_layers``).

Parity: reference ``inference/mmfp4_pipeline.py`` (``_fused_sampling`` :224 - greedy / top-k / top-p / plain sampling in one call,
``_optimized_generate`` :428 - preallocated buffers, no per-step concatenation).
"""
from __future__ import annotations

from typing import Any, Optional, Tuple, Union

import torch

from ..sampler import Sampler, SamplingConfig

_SAMPLERS = {}


def _fused_sampling(probs: torch.Tensor, temperature: float = 1.0, top_p: float = 0.9, top_k: int = 0, out: Optional[torch.Tensor] = None,
                    seed: Optional[int] = None, **_buffers) -> torch.Tensor:
    """Token ids ``[B, 1]`` from probabilities ``[B, V]``: arg-max when ``temperature <= 0``, else temperature, top-k and nucleus
    truncation and the draw in one sampling-kernel call (``log(probs)`` are its logits).  ``out`` (``[B, 1]`` int64) is filled when
    given.  Scratch-buffer keyword arguments of the reference signature are accepted and unused: the kernel works in place."""
    if probs.dim() == 1:
        probs = probs.unsqueeze(0)
    key = (probs.shape[-1], str(probs.device))
    smp = _SAMPLERS.get(key)
    if smp is None:
        smp = _SAMPLERS[key] = Sampler(probs.shape[-1], probs.device)
    if temperature <= 0.0:
        ids = smp.argmax(probs.float())
    else:
        cfg = SamplingConfig(temperature=float(temperature), top_k=int(top_k), top_p=float(top_p) if 0.0 < top_p <= 1.0 else 1.0, seed=seed)
        ids = smp.sample(torch.log(probs.float().clamp_min(1e-30)), cfg)
    ids = ids.view(-1, 1).to(torch.int64)
    if out is not None:
        out.copy_(ids)
        return out
    return ids


def _optimized_generate(model: Any, input_ids: torch.Tensor, max_new_tokens: int, attention_mask: Optional[torch.Tensor] = None,
                        past_key_values: Any = None, temperature: float = 1.0, top_p: float = 0.9, top_k: int = 0, pad_token_id: Optional[int] = None,
                        eos_token_id: Optional[int] = None, return_past_key_values: bool = False, buffer_pool: Any = None, seed: Optional[int] = None
                        ) -> Union[torch.Tensor, Tuple[torch.Tensor, Any]]:
    """``[B, S] -> [B, S + n]`` (``n <= max_new_tokens``; generation stops when every row has produced ``eos_token_id``, rows that
    finished earlier are filled with ``pad_token_id``)."""
    B, S = input_ids.shape
    dev = input_ids.device
    out = torch.empty(B, S + max_new_tokens, dtype=input_ids.dtype, device=dev)
    out[:, :S] = input_ids
    mask = None
    if attention_mask is not None:
        mask = torch.ones(B, S + max_new_tokens, dtype=attention_mask.dtype, device=dev)
        mask[:, :S] = attention_mask
    finished = torch.zeros(B, dtype=torch.bool, device=dev)
    pad = pad_token_id if pad_token_id is not None else (eos_token_id if eos_token_id is not None else 0)
    nxt = torch.empty(B, 1, dtype=torch.int64, device=dev)
    cur, n = input_ids, 0
    with torch.no_grad():
        for step in range(max_new_tokens):
            kw = {"input_ids": cur, "past_key_values": past_key_values, "use_cache": True}
            if mask is not None:
                kw["attention_mask"] = mask[:, : S + step]
            res = model(**kw)
            logits = res.logits if hasattr(res, "logits") else res[0]
            past_key_values = getattr(res, "past_key_values", None) if hasattr(res, "logits") else (res[1] if len(res) > 1 else None)
            last = logits[:, -1, :].float()
            if temperature <= 0.0:
                _fused_sampling(last, 0.0, out=nxt)
            else:
                _fused_sampling(torch.softmax(last, -1), temperature, top_p, top_k, out=nxt, seed=seed)
            tok = nxt[:, 0].to(out.dtype)
            if eos_token_id is not None:
                tok = torch.where(finished, torch.full_like(tok, pad), tok)
                finished = finished | (tok == eos_token_id)
            out[:, S + step] = tok
            n = step + 1
            cur = out[:, S + step: S + step + 1] if past_key_values is not None else out[:, : S + step + 1]
            if eos_token_id is not None and bool(finished.all()):
                break
    seq = out[:, : S + n]
    return (seq, past_key_values) if return_past_key_values else seq
