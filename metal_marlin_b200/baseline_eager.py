"""Same-box baseline: the model run as plain PyTorch eager ops with bf16 library GEMMs.

``EagerBF16Model`` wraps a :class:`Transformer` and runs every op through the PyTorch restatement
(``ops/reference.py``) with the weights de-quantized once to bf16, so matrix products are cuBLAS bf16 GEMMs,
attention is gather + softmax in PyTorch, the MoE is a loop over the selected experts and every kernel is
launched from Python without a CUDA graph.  None of this package's CUDA kernels run on this path; it is what
``bench.py --impl eager`` times to show what the hand-written kernels buy on the same GPU.

Parity: the reference's own pipeline is this kind of program (PyTorch eager around per-op kernel dispatches,
``metal_marlin/inference/mmfp4_pipeline.py:428``).
"""
from __future__ import annotations

import contextlib

import torch

from . import ops
from .ops import reference as ref


@contextlib.contextmanager
def _eager_bf16():
    old = ref.MATMUL_DTYPE
    ref.MATMUL_DTYPE = torch.bfloat16
    try:
        with ops.force_reference():
            yield
    finally:
        ref.MATMUL_DTYPE = old


class EagerBF16Model:
    """Duck-types the parts of ``Transformer`` that prefill and ``DecodeSession`` use."""

    def __init__(self, model):
        self.inner = model
        self.cfg = model.cfg
        self.device = model.device
        self.tp = None

    def forward(self, *a, **kw):
        with _eager_bf16():
            return self.inner.forward(*a, **kw)

    def full_logits(self, logits):
        return logits

    def greedy(self, logits, out=None):
        r = logits.argmax(-1)
        if out is not None:
            out.copy_(r)
            return out
        return r

    def weight_bytes(self) -> int:
        return self.inner.weight_bytes()

    def prefill(self, kv, prompts, block_tables):
        from .models.mmfp4_causal_lm import prefill
        return prefill(self, kv, prompts, block_tables)
