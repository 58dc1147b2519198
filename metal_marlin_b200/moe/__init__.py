"""Mixture-of-experts utilities around the kernels: expert capacity and overflow policies, predictive expert prefetching,
load tracking with the auxiliary balancing loss and gate entropy.  The routed-expert math itself lives in ``ops.moe_forward``
(``csrc/moe_*.cu``, ``csrc/gemm_sm100.cu``) and the routing profiler in ``eval/moe_routing.py``."""
from .capacity import (CapacityAnalyzer, CapacityStats, DynamicCapacity, DynamicCapacityConfig, OverflowInfo, OverflowPolicy,
                       analyze_overflow_rate, apply_overflow_policy, auto_tune_capacity, compute_expert_capacity,
                       count_expert_assignments)
from .load_balancing import ExpertLoadTracker, LoadBalancingConfig, gate_entropy, load_balance_loss
from .prefetch import ExpertPrefetcher, PrefetchConfig, PrefetchStrategy
from .router_int8 import Int8Router, Int8RouterLinear, RouterQuantConfig, measure_quantization_error, quantize_router_weights

__all__ = ["CapacityAnalyzer", "CapacityStats", "DynamicCapacity", "DynamicCapacityConfig", "OverflowInfo", "OverflowPolicy",
           "analyze_overflow_rate", "apply_overflow_policy", "auto_tune_capacity", "compute_expert_capacity", "count_expert_assignments",
           "ExpertLoadTracker", "LoadBalancingConfig", "gate_entropy", "load_balance_loss", "ExpertPrefetcher", "PrefetchConfig",
           "PrefetchStrategy", "Int8Router", "Int8RouterLinear", "RouterQuantConfig", "measure_quantization_error",
           "quantize_router_weights"]

# ---------------------------------------------------------------------------------------------- dispatch objects under the reference's names
from dataclasses import dataclass as _dataclass

import torch as _torch

from ..compat_api import MoEDispatchInfo, group_tokens_by_expert, group_tokens_by_expert_full      # noqa: E402


@_dataclass
class GPUGroupingResult:
    """Device-side grouping: token order, its inverse and the tile list (expert, first row, rows) the grouped kernels walk."""
    order: _torch.Tensor
    inverse: _torch.Tensor
    tile_expert: _torch.Tensor
    tile_row0: _torch.Tensor
    tile_rows: _torch.Tensor
    num_tiles: _torch.Tensor


class GPUExpertGrouping:
    """Counting sort of (token, slot) pairs by expert on the device (one launch of ``csrc/moe_dispatch.cu`` on a GPU, the same
    arithmetic in PyTorch elsewhere), with the tile list for ``token_tile``-row tiles."""

    def __init__(self, num_experts: int, token_tile: int = 32):
        self.num_experts, self.token_tile = num_experts, token_tile

    def group(self, expert_ids: _torch.Tensor) -> GPUGroupingResult:
        from ..compat_api import CppDispatchInfo
        d = CppDispatchInfo.build(expert_ids, self.num_experts, self.token_tile)
        return GPUGroupingResult(d.order, d.inverse, d.tile_expert, d.tile_row0, d.tile_rows, d.num_tiles)


TopKExpertGrouping = GPUExpertGrouping


def group_tokens_by_expert_gpu(expert_ids: _torch.Tensor, num_experts: int):
    return group_tokens_by_expert(expert_ids, num_experts)


group_tokens_by_expert_fast = group_tokens_by_expert_gpu
group_tokens_by_expert_gpu_optimized = group_tokens_by_expert_gpu
group_tokens_by_expert_auto = group_tokens_by_expert_gpu


def group_tokens_by_expert_full_gpu(expert_ids: _torch.Tensor, num_experts: int) -> MoEDispatchInfo:
    return group_tokens_by_expert_full(expert_ids, num_experts)


class MoEDispatcher:
    """Route-then-compute object over a :class:`layers.MMFP4MoE` (or anything with ``route`` / ``gate_up`` / ``down``): keeps
    the expert load of every call in an :class:`ExpertLoadTracker`."""

    def __init__(self, moe_layer, tracker: "ExpertLoadTracker" = None):
        self.layer = moe_layer
        self.tracker = tracker or ExpertLoadTracker(num_experts=moe_layer.num_experts)

    def __call__(self, x: _torch.Tensor) -> _torch.Tensor:
        from .. import ops
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(_torch.bfloat16).contiguous()
        ids, w = self.layer.route(x2)
        self.tracker.update(ids)
        y = ops.moe_forward(x2, self.layer.gate_up, self.layer.down, ids, w, n_shared=self.layer.num_shared, shared_base=self.layer.num_experts)
        return y.view(shape).to(x.dtype)


FusedMoEDispatcher = MoEDispatcher

__all__ += ["GPUGroupingResult", "GPUExpertGrouping", "TopKExpertGrouping", "group_tokens_by_expert_gpu", "group_tokens_by_expert_fast",
            "group_tokens_by_expert_gpu_optimized", "group_tokens_by_expert_auto", "group_tokens_by_expert_full_gpu", "MoEDispatcher",
            "FusedMoEDispatcher", "MoEDispatchInfo", "group_tokens_by_expert", "group_tokens_by_expert_full"]


def __getattr__(name: str):
    if name in ("MoERouterCpp", "RouterBatchOutput"):
        from . import fast_router
        return getattr(fast_router, name)
    if name in ("compute_expert_load", "compute_load_balancing_loss", "gather_for_experts", "scatter_expert_outputs"):
        from .. import compat_api
        return getattr(compat_api, name)
    raise AttributeError(name)


__all__ += ["MoERouterCpp", "RouterBatchOutput", "compute_expert_load", "compute_load_balancing_loss", "gather_for_experts", "scatter_expert_outputs"]
