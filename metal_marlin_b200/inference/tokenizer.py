"""Tokenizer access: HF tokenizers from a local directory when present, else a self-contained
byte-level tokenizer (no files, no network) so pipelines, servers and tests run anywhere.

Parity: the reference loads ``AutoTokenizer.from_pretrained(path, trust_remote_code=True)``
(``metal_marlin/inference/mmfp4_pipeline.py:1853``) and ships a mock tokenizer for server tests
(``metal_marlin/serving/engine.py:416``).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence


class ByteTokenizer:
    """UTF-8 bytes + 3 specials.  ids 0..255 are bytes, 256 = <bos>, 257 = <eos>, 258 = <pad>."""
    bos_token_id, eos_token_id, pad_token_id = 256, 257, 258
    vocab_size = 259
    chat_template = "byte"

    def __init__(self, vocab_size: Optional[int] = None):
        if vocab_size is not None and vocab_size >= 259:
            self.vocab_size = vocab_size

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        ids = list(text.encode("utf-8"))
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        bs = bytes(i for i in ids if 0 <= i < 256)
        return bs.decode("utf-8", errors="replace")

    def __call__(self, text, return_tensors=None, **kw):
        ids = self.encode(text)
        if return_tensors == "pt":
            import torch
            return {"input_ids": torch.tensor([ids])}
        return {"input_ids": ids}

    def apply_chat_template(self, messages: Sequence[Dict[str, str]], add_generation_prompt: bool = True,
                            tokenize: bool = False):
        parts = [f"<|{m['role']}|>\n{m['content']}\n" for m in messages]
        if add_generation_prompt:
            parts.append("<|assistant|>\n")
        text = "".join(parts)
        return self.encode(text) if tokenize else text

    def __len__(self):
        return self.vocab_size


class HashTokenizer(ByteTokenizer):
    """Byte tokenizer folded into a model's (possibly small) vocabulary; used with random-init models."""

    def __init__(self, vocab_size: int):
        self.vocab_size = vocab_size
        self.eos_token_id = vocab_size - 1
        self.bos_token_id = vocab_size - 2
        self.pad_token_id = vocab_size - 3

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        n = max(1, self.vocab_size - 3)
        ids = [b % n for b in text.encode("utf-8")]
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        return "".join(chr(32 + (i % 95)) for i in ids if i < self.vocab_size - 3)


def load_tokenizer(path: Optional[str], vocab_size: Optional[int] = None):
    """HF tokenizer when ``path`` holds tokenizer files; otherwise a byte/hash tokenizer."""
    if path and os.path.isdir(path) and any(os.path.exists(os.path.join(path, f))
                                            for f in ("tokenizer.json", "tokenizer.model", "vocab.json")):
        try:
            from transformers import AutoTokenizer
            return AutoTokenizer.from_pretrained(path, trust_remote_code=False, local_files_only=True)
        except Exception:
            pass
    if vocab_size is not None and vocab_size < 259:
        return HashTokenizer(vocab_size)
    return ByteTokenizer(vocab_size)
