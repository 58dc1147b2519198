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

    def generate(self, prompts, max_new_tokens: int = 32, **kw):
        kw.setdefault("use_graph", False)
        return super().generate(prompts, max_new_tokens=max_new_tokens, **kw)

    def bit_histogram(self, path: str):
        return TrellisModelLoader(path).bit_histogram()
