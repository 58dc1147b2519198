"""``TrellisForCausalLM``: causal LM over a trellis-quantized checkpoint (v2 layer directories or v3 HF shards).

Parity: reference ``metal_marlin/trellis/lm.py:57`` (``TrellisForCausalLM.from_pretrained``, ``forward``), config
``metal_marlin/trellis/config.py:75``, loader ``metal_marlin/trellis/loader.py:156``, linear ``trellis/linear.py:50``,
MoE ``trellis/moe.py:131``.  The reference's attention is MLA-only (it raises without ``q_a/q_b``); here the same
decoder (``models/transformer.py``: MLA or GQA attention, dense or MoE MLP, paged KV, fused sampler) runs on
``TrellisLinear`` weights through the op layer's generic-weight path, so GQA trellis models (Qwen3-style) load as
well.  Decode GEMVs read the 2-8 bit tile stream directly; prefill de-quantizes a matrix to bf16 transiently and uses
the tcgen05 bf16 GEMM.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional, Sequence

import torch

from ..formats.trellis import TrellisModelLoader
from ..layers.linear import TrellisLinear
from ..models.config import ModelConfig
from ..models.loading import build_transformer
from ..models.mmfp4_causal_lm import MMFP4ForCausalLM
from ..ops.generic import CatWeight, GenericExpertBank

TrellisModelConfig = ModelConfig      # same fields (GLM MLA / Qwen3 GQA-MoE / DeepSeek); parsed from the checkpoint's config.json


class TrellisSource:
    """Checkpoint source handing out ``TrellisLinear`` weights (see ``models/loading.py`` for the protocol)."""

    def __init__(self, cfg: ModelConfig, path: str, device):
        self.cfg, self.device = cfg, torch.device(device)
        self.loader = TrellisModelLoader(path)

    def _name(self, name: str) -> str:
        for cand in (name + ".weight", name, name.replace("model.", "model.language_model.", 1) + ".weight"):
            if self.loader.has_weight(cand):
                return cand
        raise KeyError(f"trellis checkpoint has no quantized weight {name!r}")

    def has(self, name: str) -> bool:
        return self.loader.has_tensor(name) or self.loader.has_weight(name)

    def linear(self, name: str, out_f: int, in_f: int):
        try:
            tw = self.loader.load_weight(self._name(name))
        except KeyError:
            # kept in 16 bit by the quantizer (routers, small projections): wrap as a dense generic weight
            return _DenseWeight(self.loader.load_tensor(name + ".weight").to(self.device, torch.bfloat16))
        assert tuple(tw.shape) == (out_f, in_f), (name, tw.shape, out_f, in_f)
        return TrellisLinear(tw, self.device)

    def linear_cat(self, names, outs, in_f):
        return CatWeight([self.linear(n, o, in_f) for n, o in zip(names, outs)])

    def dense(self, name: str, *shape, std=None) -> torch.Tensor:
        t = self.loader.load_tensor(name).to(self.device, torch.bfloat16)
        assert tuple(t.shape) == tuple(shape), (name, t.shape, shape)
        return t

    def norm(self, name: str, dim: int) -> torch.Tensor:
        return self.dense(name, dim)

    def float(self, name: str, *shape, std=None) -> torch.Tensor:
        return self.loader.load_tensor(name).to(self.device, torch.float32)

    def expert_banks(self, m: str, E: int, I: int, H: int, ns: int):
        gus, dws = [], []
        for e in range(E):
            p = f"{m}.experts.{e}"
            gus.append(self.linear_cat([f"{p}.gate_proj", f"{p}.up_proj"], [I, I], H))
            dws.append(self.linear(f"{p}.down_proj", H, I))
        if ns:
            p = f"{m}.shared_experts"
            gus.append(self.linear_cat([f"{p}.gate_proj", f"{p}.up_proj"], [ns * I, ns * I], H))
            dws.append(self.linear(f"{p}.down_proj", H, ns * I))
            gus.extend([None] * (ns - 1))
            dws.extend([None] * (ns - 1))
        bank = GenericExpertBank(gus, dws)
        return bank, bank


class TrellisRandomSource:
    """Random-init trellis weights of an architecture preset (synthetic benchmarks): attention and dense matrices at
    ``dense_bits``, expert ``e`` at ``expert_bits[e % len(expert_bits)]`` (mixed precision per expert, as the trellis-v2
    quantizer assigns it), routers / norms / embeddings in bf16.  Every rank of a multi-GPU job draws the same tensors."""

    def __init__(self, cfg: ModelConfig, device, seed: int = 0, dense_bits: int = 4, expert_bits=(2, 3, 4), group_size: int = 128):
        self.cfg, self.device, self.seed = cfg, torch.device(device), seed
        self.dense_bits, self.expert_bits, self.gs = dense_bits, tuple(expert_bits), group_size

    def _seed(self, name: str) -> int:
        import zlib
        return (zlib.crc32(name.encode()) + self.seed * 7919) & 0x7FFFFFFF

    def _gs(self, in_f: int) -> int:
        gs = self.gs
        while gs > 16 and in_f % gs:
            gs //= 2
        return gs

    def has(self, name: str) -> bool:
        return True

    def linear(self, name: str, out_f: int, in_f: int, bits: Optional[int] = None):
        return TrellisLinear.random(out_f, in_f, bits or self.dense_bits, self._gs(in_f), self.device, self._seed(name))

    def linear_cat(self, names, outs, in_f):
        return CatWeight([self.linear(n, o, in_f) for n, o in zip(names, outs)])

    def dense(self, name: str, *shape, std=None) -> torch.Tensor:
        g = torch.Generator(device=self.device).manual_seed(self._seed(name))
        return (torch.randn(*shape, device=self.device, generator=g) * (std or 0.02)).to(torch.bfloat16)

    def norm(self, name: str, dim: int) -> torch.Tensor:
        return torch.ones(dim, dtype=torch.bfloat16, device=self.device)

    def float(self, name: str, *shape, std=None) -> torch.Tensor:
        g = torch.Generator(device=self.device).manual_seed(self._seed(name))
        return torch.randn(*shape, device=self.device, generator=g) * (std or 0.02)

    def expert_banks(self, m: str, E: int, I: int, H: int, ns: int):
        gus, dws = [], []
        for e in range(E):
            b = self.expert_bits[e % len(self.expert_bits)]
            p = f"{m}.experts.{e}"
            gus.append(CatWeight([self.linear(f"{p}.gate_proj", I, H, b), self.linear(f"{p}.up_proj", I, H, b)]))
            dws.append(self.linear(f"{p}.down_proj", H, I, b))
        for j in range(ns):
            p = f"{m}.shared_experts.{j}"
            gus.append(CatWeight([self.linear(f"{p}.gate_proj", I, H), self.linear(f"{p}.up_proj", I, H)]))
            dws.append(self.linear(f"{p}.down_proj", H, I))
        bank = GenericExpertBank(gus, dws)
        return bank, bank


class _DenseWeight:
    is_generic = True
    names = None

    def __init__(self, w: torch.Tensor):
        self.w = w
        self.out_features, self.in_features = w.shape

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        from ..layers.linear import _bf16_matmul
        return _bf16_matmul(x.contiguous(), self.w)

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        return self.w.to(dtype)


class TrellisForCausalLM(MMFP4ForCausalLM):
    """Same public surface as ``MMFP4ForCausalLM`` (``generate``, ``forward_logits``, ``new_cache``); decode runs
    eagerly (the expert loop reads routing on the host)."""

    @classmethod
    def from_pretrained(cls, path: str, device: Optional[str] = None) -> "TrellisForCausalLM":
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        cfg = ModelConfig.from_pretrained(path)
        return cls(build_transformer(cfg, TrellisSource(cfg, path, device)))

    @classmethod
    def from_config(cls, cfg, device: Optional[str] = None, seed: int = 0, dense_bits: int = 4, expert_bits=(2, 3, 4)) -> "TrellisForCausalLM":
        """Random-init trellis model of an architecture preset (see :class:`TrellisRandomSource`)."""
        from ..models.config import get_preset
        if isinstance(cfg, str):
            cfg = get_preset(cfg)
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        return cls(build_transformer(cfg, TrellisRandomSource(cfg, device, seed, dense_bits, expert_bits)))

    def generate(self, prompts, max_new_tokens: int = 32, **kw):
        kw.setdefault("use_graph", False)
        return super().generate(prompts, max_new_tokens=max_new_tokens, **kw)

    def bit_histogram(self, path: str):
        return TrellisModelLoader(path).bit_histogram()
