"""Device mesh: maps the ranks of a job onto (dp, pp, tp) coordinates - expert parallelism reuses the tp axis - and
creates the process group of every axis.

Parity: reference ``metal_marlin/distributed/device_mesh.py`` (a simulated mesh of logical devices); here the ranks
are real processes, one per GPU, and the groups are NCCL (or gloo on CPU) communicators.  Layout: tp is the
fastest-varying axis so that a tp group sits on NVLink-adjacent GPUs of one node, then pp, then dp.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch.distributed as dist


@dataclass(frozen=True)
class MeshShape:
    dp: int = 1
    pp: int = 1
    tp: int = 1

    @property
    def world(self) -> int:
        return self.dp * self.pp * self.tp


class DeviceMesh:
    def __init__(self, shape: MeshShape, rank: Optional[int] = None, create_groups: bool = True):
        self.shape = shape
        self.rank = dist.get_rank() if rank is None else rank
        if create_groups and dist.is_initialized() and dist.get_world_size() != shape.world:
            raise ValueError(f"mesh {shape} needs {shape.world} ranks, the job has {dist.get_world_size()}")
        self.groups: Dict[str, Optional[dist.ProcessGroup]] = {"dp": None, "pp": None, "tp": None}
        if create_groups and dist.is_initialized():
            for axis in ("tp", "pp", "dp"):
                for members in self.all_groups(axis):       # every rank must take part in every new_group call
                    g = dist.new_group(members)
                    if self.rank in members:
                        self.groups[axis] = g

    def coords(self, rank: Optional[int] = None) -> Tuple[int, int, int]:
        """(dp, pp, tp) coordinates of a rank."""
        r = self.rank if rank is None else rank
        s = self.shape
        return r // (s.pp * s.tp), (r // s.tp) % s.pp, r % s.tp

    def rank_of(self, dp: int, pp: int, tp: int) -> int:
        s = self.shape
        return (dp * s.pp + pp) * s.tp + tp

    def all_groups(self, axis: str) -> List[List[int]]:
        s = self.shape
        out = []
        if axis == "tp":
            for d in range(s.dp):
                for p in range(s.pp):
                    out.append([self.rank_of(d, p, t) for t in range(s.tp)])
        elif axis == "pp":
            for d in range(s.dp):
                for t in range(s.tp):
                    out.append([self.rank_of(d, p, t) for p in range(s.pp)])
        elif axis == "dp":
            for p in range(s.pp):
                for t in range(s.tp):
                    out.append([self.rank_of(d, p, t) for d in range(s.dp)])
        else:
            raise ValueError(axis)
        return out

    def group_ranks(self, axis: str) -> List[int]:
        return next(g for g in self.all_groups(axis) if self.rank in g)

    def group(self, axis: str):
        return self.groups[axis]

    def pp_neighbours(self) -> Tuple[Optional[int], Optional[int]]:
        d, p, t = self.coords()
        prev = self.rank_of(d, p - 1, t) if p > 0 else None
        nxt = self.rank_of(d, p + 1, t) if p + 1 < self.shape.pp else None
        return prev, nxt


def plan_mesh(world: int, model_bytes: float, hbm_bytes: float = 180e9, kv_bytes: float = 0.0, prefer: str = "dp") -> MeshShape:
    """Smallest tp x pp product whose weight shard (plus KV budget) fits one GPU; the remaining ranks become data-parallel
    replicas.  ``prefer='tp'`` spends every rank on tensor parallelism (latency mode)."""
    if prefer == "tp":
        return MeshShape(1, 1, world)
    need = 1
    while need < world and (model_bytes / need + kv_bytes) > 0.9 * hbm_bytes:
        need *= 2
    if (model_bytes / need + kv_bytes) > 0.9 * hbm_bytes:
        raise ValueError(f"model of {model_bytes / 1e9:.0f} GB does not fit {world} GPUs of {hbm_bytes / 1e9:.0f} GB")
    tp = min(need, 8)
    pp = need // tp
    return MeshShape(world // (tp * pp), pp, tp)
