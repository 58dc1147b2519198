"""Multi-GPU: tensor / expert / pipeline / context parallelism, the device mesh, the symmetric-memory runtime and health
monitoring, plus functional collectives and sharding helpers under the names of the reference's ``metal_marlin.distributed``
package (parity: its ``__init__`` exports ``Device`` / ``DeviceType`` / ``DeviceMesh``, ``ParallelMode``, ``ShardSpec`` /
``shard_tensor``, ``TensorParallelLinear``, ``PipelineConfig`` / ``PipelineParallel``, ``all_reduce`` / ``all_gather`` / ``broadcast`` /
``scatter``; the reference simulates devices in one process, here every rank is a process on its own GPU and the collectives
are ``torch.distributed`` calls that degrade to the identity without a process group)."""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .health import (DeviceWaitExpired, ExpertCapacityOverflow, Heartbeat, PeerFailure, StepGuard, decode_status, make_heartbeat,
                     raise_for_status)
from .mesh import DeviceMesh, MeshShape, plan_mesh


class DeviceType(enum.Enum):
    CUDA = "cuda"
    CPU = "cpu"


@dataclass
class Device:
    index: int
    type: DeviceType = DeviceType.CUDA
    name: str = ""
    total_memory: int = 0

    @classmethod
    def discover(cls) -> List["Device"]:
        if not torch.cuda.is_available():
            return [cls(0, DeviceType.CPU, "cpu", 0)]
        return [cls(i, DeviceType.CUDA, torch.cuda.get_device_name(i), torch.cuda.get_device_properties(i).total_memory)
                for i in range(torch.cuda.device_count())]

    @property
    def torch_device(self) -> torch.device:
        return torch.device("cpu") if self.type is DeviceType.CPU else torch.device("cuda", self.index)


class ParallelMode(enum.Enum):
    NONE = "none"
    COLUMN = "column"        # output features split: each rank computes a slice of the output
    ROW = "row"              # input features split: partial sums are added across the ranks


@dataclass
class ShardSpec:
    dim: int
    rank: int
    world: int
    unit: int = 1            # slices are multiples of this many elements (quantization groups, tiles)

    def bounds(self, size: int):
        from .tp import even_split
        return even_split(size, self.world, self.unit)[self.rank]


def shard_tensor(t: torch.Tensor, dim: int, rank: int, world: int, unit: int = 1) -> torch.Tensor:
    """The ``rank``-th of ``world`` near-equal slices of ``t`` along ``dim`` (slice sizes multiples of ``unit``)."""
    a, b = ShardSpec(dim, rank, world, unit).bounds(t.shape[dim])
    return t.narrow(dim, a, b - a).contiguous()


def _group_ok(group=None) -> bool:
    import torch.distributed as dist
    return dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1


def all_reduce(t: torch.Tensor, group=None, op: str = "sum") -> torch.Tensor:
    import torch.distributed as dist
    if _group_ok(group):
        dist.all_reduce(t, op={"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[op], group=group)
    return t


def all_gather(t: torch.Tensor, group=None, dim: int = 0) -> torch.Tensor:
    import torch.distributed as dist
    if not _group_ok(group):
        return t
    parts = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.cat(parts, dim)


def broadcast(t: torch.Tensor, src: int = 0, group=None) -> torch.Tensor:
    import torch.distributed as dist
    if _group_ok(group):
        dist.broadcast(t, src=src, group=group)
    return t


def scatter(t: Optional[torch.Tensor], src: int = 0, group=None, dim: int = 0) -> torch.Tensor:
    """Rank ``src`` holds the whole tensor; every rank gets its slice along ``dim``."""
    import torch.distributed as dist
    if not _group_ok(group):
        return t
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    meta = [None]
    if rank == src:
        meta = [(tuple(t.shape), t.dtype)]
    dist.broadcast_object_list(meta, src=src, group=group)
    shape, dtype = meta[0]
    per = list(shape)
    per[dim] //= world
    out = torch.empty(per, dtype=dtype, device=t.device if t is not None else None)
    chunks = [c.contiguous() for c in t.chunk(world, dim)] if rank == src else None
    dist.scatter(out, chunks, src=src, group=group)
    return out


class TensorParallelLinear:
    """A float or FP4 linear split over the ranks of ``group``: ``COLUMN`` keeps a slice of the output features (results are
    gathered when ``gather_output``), ``ROW`` a slice of the input features (partial sums are all-reduced)."""

    def __init__(self, weight: torch.Tensor, mode: ParallelMode = ParallelMode.COLUMN, rank: int = 0, world: int = 1, group=None,
                 bias: Optional[torch.Tensor] = None, gather_output: bool = True, quantize: bool = False, group_size: int = 128):
        self.mode, self.rank, self.world, self.group, self.gather_output = mode, rank, world, group, gather_output
        unit = group_size if quantize else 1
        if mode is ParallelMode.COLUMN:
            w = shard_tensor(weight, 0, rank, world, 16 if quantize else 1)
            self.bias = None if bias is None else shard_tensor(bias, 0, rank, world, 16 if quantize else 1)
        elif mode is ParallelMode.ROW:
            w = shard_tensor(weight, 1, rank, world, max(unit, 64) if quantize else 1)
            self.bias = bias if rank == 0 else None
            self.in_bounds = ShardSpec(1, rank, world, max(unit, 64) if quantize else 1).bounds(weight.shape[1])
        else:
            w, self.bias = weight, bias
        if quantize:
            from ..layers.linear import MMFP4Linear
            self.inner = MMFP4Linear.from_float(w.float(), group_size, device=w.device)
        else:
            self.inner = None
            self.weight = w

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.mode is ParallelMode.ROW and x.shape[-1] != (self.inner.in_features if self.inner is not None else self.weight.shape[1]):
            a, b = self.in_bounds
            x = x[..., a:b]
        y = self.inner(x) if self.inner is not None else torch.nn.functional.linear(x, self.weight.to(x.dtype))
        if self.mode is ParallelMode.ROW:
            y = all_reduce(y.contiguous(), self.group)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        if self.mode is ParallelMode.COLUMN and self.gather_output:
            y = all_gather(y, self.group, dim=-1)
        return y


@dataclass
class PipelineConfig:
    num_stages: int = 1
    num_microbatches: int = 1
    overlap: bool = True


class PipelineParallel:
    """Splits a layer list over pipeline stages and runs micro-batches through this rank's stage (``parallel/pp.py``)."""

    def __init__(self, num_layers: int, config: Optional[PipelineConfig] = None, rank: int = 0):
        from .pp import stage_layers
        self.config = config or PipelineConfig()
        self.rank = rank
        self.stages = stage_layers(num_layers, self.config.num_stages)

    @property
    def my_layers(self) -> range:
        a, b = self.stages[self.rank]
        return range(a, b)

    def stage_of(self, layer: int) -> int:
        return next(i for i, (a, b) in enumerate(self.stages) if a <= layer < b)


def __getattr__(name: str):
    lazy = {"TPContext": (".tp", "TPContext"), "shard_transformer": (".tp", "shard_transformer"), "make_context": (".tp", "make_context"),
            "even_split": (".tp", "even_split"), "ExpertParallelMoE": (".ep", "ExpertParallelMoE"), "EPExchange": (".ep", "EPExchange"),
            "shard_transformer_ep": (".ep", "shard_transformer_ep"), "expert_range": (".ep", "expert_range"),
            "PipelineStage": (".pp", "PipelineStage"), "pipeline_prefill": (".pp", "pipeline_prefill"),
            "pipeline_decode_step": (".pp", "pipeline_decode_step"), "stage_layers": (".pp", "stage_layers"),
            "ring_attention": (".cp", "ring_attention"), "SymmetricBuffer": (".symm", "SymmetricBuffer")}
    if name in lazy:
        import importlib
        mod, attr = lazy[name]
        return getattr(importlib.import_module(mod, __package__), attr)
    raise AttributeError(name)


__all__ = ["Device", "DeviceType", "DeviceMesh", "MeshShape", "plan_mesh", "ParallelMode", "ShardSpec", "shard_tensor", "TensorParallelLinear",
           "PipelineConfig", "PipelineParallel", "all_reduce", "all_gather", "broadcast", "scatter", "PeerFailure", "DeviceWaitExpired",
           "ExpertCapacityOverflow", "Heartbeat", "StepGuard", "decode_status", "make_heartbeat", "raise_for_status", "TPContext",
           "shard_transformer", "make_context", "even_split", "ExpertParallelMoE", "EPExchange", "shard_transformer_ep", "expert_range",
           "PipelineStage", "pipeline_prefill", "pipeline_decode_step", "stage_layers", "ring_attention", "SymmetricBuffer"]
