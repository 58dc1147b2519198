"""Expert parallelism.

Two regimes:

* decode (few tokens, replicated on every rank of the group because attention is replicated or tensor parallel): no
  token ever moves.  Every rank runs the routed experts it owns for all tokens - remote experts are masked to id -1,
  which the MoE kernels skip - and the partial outputs are summed with the same in-kernel NVLink exchange the
  tensor-parallel row projections use (``csrc/tp_comm.cuh``): dispatch is implicit, combine is fused into the
  down-projection epilogue.
* prefill / large batches: tokens are sent to the ranks owning their experts (all-to-all), run through the grouped
  tcgen05 expert GEMM there and returned (all-to-all), the NCCL baseline.

Parity: reference ``metal_marlin/distributed/expert_parallel.py`` (simulated expert placement + dispatch / combine).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..ops.weights import FP4ExpertBank


def expert_range(num_experts: int, rank: int, ep: int) -> Tuple[int, int]:
    per = (num_experts + ep - 1) // ep
    return min(num_experts, rank * per), min(num_experts, (rank + 1) * per)


def shard_bank(bank: FP4ExpertBank, num_routed: int, n_shared: int, rank: int, ep: int) -> Tuple[FP4ExpertBank, int, int, int]:
    """Local bank = this rank's routed experts, followed by the shared experts on rank 0 only.  Returns
    ``(bank, first_expert, n_local_routed, n_local_shared)``."""
    e0, e1 = expert_range(num_routed, rank, ep)
    idx = list(range(e0, e1)) + (list(range(num_routed, num_routed + n_shared)) if rank == 0 else [])
    sel = torch.tensor(idx, dtype=torch.long, device=bank.qtile.device)
    local = FP4ExpertBank(bank.qtile.index_select(0, sel).contiguous(), bank.stile.index_select(0, sel).contiguous(),
                          bank.out_features, bank.in_features, bank.group_size)
    return local, e0, e1 - e0, (n_shared if rank == 0 else 0)


def localize_ids(ids: torch.Tensor, first: int, n_local: int) -> torch.Tensor:
    """Global expert ids -> local ids, -1 for experts other ranks own (no host sync)."""
    loc = ids.to(torch.int32) - first
    return torch.where((loc >= 0) & (loc < n_local), loc, torch.full_like(loc, -1))


class ExpertParallelMoE:
    """One MoE layer's experts sharded over the ranks of ``group``."""

    def __init__(self, gate_up: FP4ExpertBank, down: FP4ExpertBank, num_routed: int, n_shared: int, rank: int, ep: int, group=None):
        self.rank, self.ep, self.group = rank, ep, group
        self.num_routed = num_routed
        self.gate_up, self.first, self.n_local, self.n_shared_local = shard_bank(gate_up, num_routed, n_shared, rank, ep)
        self.down = shard_bank(down, num_routed, n_shared, rank, ep)[0]

    def partial(self, x, ids, weights, *, norm_w=None, eps=1e-6, tpx=None):
        """This rank's share of the expert output for replicated tokens (sum over ranks = full MoE output)."""
        lid = localize_ids(ids, self.first, self.n_local)
        return ops.moe_forward(x, self.gate_up, self.down, lid, weights, n_shared=self.n_shared_local, shared_base=self.n_local,
                               norm_w=norm_w, eps=eps, tpx=tpx)

    def forward_replicated(self, x, ids, weights, *, norm_w=None, eps=1e-6):
        """Decode regime with a library collective (baseline; the fused path passes ``tpx`` to :meth:`partial`)."""
        y = self.partial(x, ids, weights, norm_w=norm_w, eps=eps).to(torch.float32)
        if self.ep > 1:
            dist.all_reduce(y, group=self.group)
        return y.to(torch.bfloat16)

    def forward_dispatch(self, x_local, ids_local, weights_local, *, norm_w=None, eps=1e-6):
        """Prefill regime: every rank holds different tokens ``x_local [T_r, H]``.  Tokens travel to expert owners and back."""
        ep, dev = self.ep, x_local.device
        xin = ops.rmsnorm(x_local, norm_w, eps) if norm_w is not None else x_local
        T, k = ids_local.shape
        flat_e = ids_local.reshape(-1).long()
        owner = torch.div(flat_e, (self.num_routed + ep - 1) // ep, rounding_mode="floor").clamp_(0, ep - 1)
        order = torch.argsort(owner, stable=True)
        send_counts = torch.bincount(owner, minlength=ep)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        tok = torch.div(order, k, rounding_mode="floor")
        send_x = xin.index_select(0, tok).contiguous()
        send_e = flat_e.index_select(0, order).contiguous()
        recv_x = torch.empty(sum(rc), xin.shape[1], dtype=xin.dtype, device=dev)
        recv_e = torch.empty(sum(rc), dtype=torch.long, device=dev)
        dist.all_to_all_single(recv_x, send_x, rc, sc, group=self.group)
        dist.all_to_all_single(recv_e, send_e, rc, sc, group=self.group)
        # local experts on the received (token, expert) pairs: one slot per row, weight 1 (weights applied at home)
        lid = localize_ids(recv_e.view(-1, 1), self.first, self.n_local)
        ones = torch.ones(recv_x.shape[0], 1, dtype=torch.float32, device=dev)
        y = ops.moe_forward(recv_x, self.gate_up, self.down, lid, ones) if recv_x.shape[0] else recv_x.new_zeros(0, self.down.out_features)
        back = torch.empty(send_x.shape[0], self.down.out_features, dtype=y.dtype, device=dev)
        dist.all_to_all_single(back, y.contiguous(), sc, rc, group=self.group)
        w_sorted = weights_local.reshape(-1).index_select(0, order).to(torch.float32)
        out = torch.zeros(T, self.down.out_features, dtype=torch.float32, device=dev)
        out.index_add_(0, tok, back.to(torch.float32) * w_sorted.unsqueeze(-1))
        return out.to(torch.bfloat16)
