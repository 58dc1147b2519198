"""Per-row LoRA adapters on top of a quantized base projection: every row of a batch names its adapter (``-1`` = none), the
base product runs once for the whole batch on the quantized kernels, and the low-rank terms are added adapter by adapter
over the rows that use them (rows are grouped by adapter first, so each adapter costs two small dense products whatever
the order of the batch).

``LoRAMixin.batch_aware_dispatch`` is mixed into the linear layer classes.  Reference ``layers/mixed_precision_linear.py:183`` and
``MarlinLinear.batch_aware_dispatch`` (``tests/test_batch_aware_lora.py``).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch

Adapters = Union[torch.Tensor, Sequence[torch.Tensor], None]


def apply_lora(out: torch.Tensor, x: torch.Tensor, lora_u: Adapters, lora_v: Adapters, lora_indices: Optional[torch.Tensor],
               scaling: float = 1.0) -> torch.Tensor:
    """``out[t] += scaling * (x[t] @ U[a]) @ V[a]`` with ``a = lora_indices[t]`` (skipped for ``a < 0``).  ``lora_u``: ``[A, in, r]`` or a list of
    ``[in, r_a]`` (ranks may differ in a list); ``lora_v``: ``[A, r, out]`` or a list of ``[r_a, out]``.  ``lora_indices`` has one entry per
    leading row of ``x`` (``[batch]`` for ``x [batch, ..., in]``: all tokens of a sequence share its adapter) or per flattened row.
    Returns ``out`` (updated in place when it is a float tensor of the accumulation dtype)."""
    if lora_u is None or lora_v is None or lora_indices is None:
        return out
    xf = x.reshape(-1, x.shape[-1])
    of = out.reshape(-1, out.shape[-1])
    idx = lora_indices.reshape(-1).to(xf.device)
    rows = xf.shape[0]
    if idx.numel() != rows:
        if rows % idx.numel():
            raise ValueError(f"{idx.numel()} adapter indices for {rows} rows")
        idx = idx.repeat_interleave(rows // idx.numel())
    n_adapters = len(lora_u)
    if int(idx.max()) >= n_adapters:
        raise ValueError(f"adapter index {int(idx.max())} out of range [0, {n_adapters})")
    order = torch.argsort(idx, stable=True)
    sorted_idx = idx[order]
    present, counts = torch.unique_consecutive(sorted_idx, return_counts=True)
    start = 0
    for a, n in zip(present.tolist(), counts.tolist()):
        sel = order[start: start + n]
        start += n
        if a < 0:
            continue
        u, v = lora_u[a].to(xf.device), lora_v[a].to(xf.device)
        acc = torch.promote_types(xf.dtype, u.dtype) if xf.is_floating_point() else u.dtype
        delta = (xf[sel].to(acc) @ u.to(acc)) @ v.to(acc)
        of.index_add_(0, sel, (scaling * delta).to(of.dtype))
    return out


class LoRAMixin:
    def batch_aware_dispatch(self, x: torch.Tensor, lora_u: Adapters = None, lora_v: Adapters = None, lora_indices: Optional[torch.Tensor] = None,
                             scaling: float = 1.0) -> torch.Tensor:
        """The layer's output with per-row LoRA terms added (see :func:`apply_lora`)."""
        out = self(x)
        if lora_u is None or lora_v is None or lora_indices is None:
            return out
        return apply_lora(out.clone() if out.data_ptr() == x.data_ptr() else out, x, lora_u, lora_v, lora_indices, scaling)
