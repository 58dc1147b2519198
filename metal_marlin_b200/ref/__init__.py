"""CPU oracles implemented natively (``csrc/runtime.cpp``): independent restatements of the router, the logits
processing order of the sampler, FP4 / codebook de-quantization, MoE token grouping and 2:4 pruning, used by tests to
check the CUDA kernels and the PyTorch restatements against a third implementation.

Parity: reference ``cpp/src/moe_router_dispatch.cpp``, ``metal_marlin/cpp/logits_ops.hpp``,
``metal_marlin/utils/cpu_dequant.cpp``, ``cpp/src/moe_manager.mm``, ``cpp/src/weights_ops.cpp``."""
from __future__ import annotations

import torch

from .. import _build


def _n():
    _build.load(require=True)
    return torch.ops.mmb200


def dequant_fp4(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    return _n().cpu_dequant_fp4(codes.cpu(), scales.cpu())


def dequant_codebook(codes, scales, zeros, lut) -> torch.Tensor:
    return _n().cpu_dequant_codebook(codes.cpu(), scales.cpu(), None if zeros is None else zeros.cpu(), lut.cpu())


def router_topk(x, w, bias=None, topk=4, scoring=0, renorm=True, routed_scale=1.0):
    return _n().cpu_router_topk(x.cpu(), w.cpu(), None if bias is None else bias.cpu(), topk, scoring, renorm, routed_scale)


def logits_process(logits, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, rep_penalty=1.0, history=None) -> torch.Tensor:
    return _n().cpu_logits_process(logits.cpu(), temperature, top_k, top_p, min_p, rep_penalty, None if history is None else history.cpu())


def group_tokens(ids, num_experts):
    return _n().cpu_group_tokens(ids.cpu(), num_experts)


def plan_grouped_gemm(counts, offsets, expert_bits, token_tile=64) -> torch.Tensor:
    return _n().plan_grouped_gemm(counts.cpu(), offsets.cpu(), expert_bits.cpu(), token_tile)


def prune_2_4(w):
    return _n().prune_2_4(w.cpu())
