"""Symmetric (peer-addressable) device memory for the in-kernel NVLink exchange.

One allocation per rank with the same layout on every rank; after the rendezvous every rank knows the
device address of every peer's copy, so kernels can store into / load from peer memory directly.

Backends (``MMB200_SYMM_BACKEND`` = ``vmm`` | ``torch`` | ``ipc``; default: ``vmm``, then ``torch``, then ``ipc`` when the
one before raises):

* ``vmm``: this library's own allocator (``csrc/symm_vmm.cpp``): a physical allocation created with the CUDA virtual-memory
  API, exported as a file descriptor, passed to the peers over Unix sockets (``SCM_RIGHTS``), imported and mapped by each of
  them; bound to an NVSwitch multicast object created by rank 0 (unless ``MMB200_SYMM_MULTICAST=0`` or NVLS is switched
  off with ``NCCL_NVLS_ENABLE=0``), whose mapping is the ``multimem`` address of all copies.  No private PyTorch API is
  involved.
* ``torch``: ``torch.distributed._symmetric_memory`` (the same mechanism inside PyTorch; multicast where the fabric has it).
* ``ipc``: CUDA IPC handles of a regular torch allocation exchanged through the process group (no multicast).

Parity: nothing comparable exists in the reference (its "collectives" are numpy concatenations inside one
process, ``metal_marlin/distributed/tensor_parallel.py:142-276``); this module is the communication runtime
the B200 build needs for its fused tensor-parallel kernels.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


class SymmetricBuffer:
    """``nbytes`` of zero-initialised device memory on every rank of ``group`` + all peers' addresses."""

    def __init__(self, nbytes: int, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.device = device
        self.nbytes = (nbytes + 255) // 256 * 256
        self.backend = None
        self._handle = None
        self.multicast_ptr = 0
        self._peer_tensors: List[torch.Tensor] = []
        err = None
        import os
        want = os.environ.get("MMB200_SYMM_BACKEND", "")
        mc = os.environ.get("MMB200_SYMM_MULTICAST", "1") != "0" and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0"
        order = {"vmm": ["vmm"], "torch": ["torch", "ipc"], "ipc": ["ipc"]}.get(want, ["vmm", "torch", "ipc"])
        for i, be in enumerate(order):
            try:
                if be == "vmm":
                    self._init_vmm(mc)              # without multicast on the fabric: peer pointers only (multicast_ptr 0)
                    self.backend = "vmm"
                elif be == "torch":
                    self._init_symm_mem()
                    self.backend = "symmetric_memory"
                else:
                    self._init_ipc()
                    self.backend = "cuda_ipc"
                break
            except Exception as e:
                err = e
                if i == len(order) - 1:
                    raise
        self.init_error = repr(err) if err else None
        self.local.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(self.group)

    # ------------------------------------------------------------------ backends
    def _init_symm_mem(self) -> None:
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        hdl = symm_mem.rendezvous(t, self.group.group_name if hasattr(self.group, "group_name") else self.group)
        self.local = t
        self._handle = hdl
        self.peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
        # address of the same allocation through the NVSwitch multicast object (0 when the fabric or the driver has none):
        # a multimem store there lands in every rank's copy
        self.multicast_ptr = int(getattr(hdl, "multicast_ptr", 0) or 0)
        assert len(self.peer_ptrs) == self.world and self.peer_ptrs[self.rank] == t.data_ptr()

    def _init_vmm(self, multicast: bool) -> None:
        from .vmm import VmmExchange
        self._vmm = VmmExchange(self.nbytes, self.device, self.group, multicast=multicast)
        self.local = self._vmm.local
        self.peer_ptrs = list(self._vmm.peer_ptrs)
        self.multicast_ptr = self._vmm.multicast_ptr
        self.nbytes = self._vmm.nbytes

    def close(self) -> None:
        """Unmap and release what the own allocator holds (the other backends free with their tensors)."""
        v = getattr(self, "_vmm", None)
        if v is not None:
            v.close()
            self._vmm = None

    def _init_ipc(self) -> None:
        t = torch.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        st = t.untyped_storage()
        meta = st._share_cuda_()
        gathered = [None] * self.world
        dist.all_gather_object(gathered, (meta, t.storage_offset()), group=self.group)
        self.local = t
        self.peer_ptrs = []
        for r, (m, off) in enumerate(gathered):
            if r == self.rank:
                self.peer_ptrs.append(t.data_ptr())
                continue
            ps = torch.UntypedStorage._new_shared_cuda(*m)
            pt = torch.empty(0, dtype=torch.uint8, device=ps.device).set_(ps, off, (self.nbytes,))
            self._peer_tensors.append(pt)
            # make sure peer access is enabled between the two devices (a copy triggers torch's P2P setup)
            probe = torch.empty(16, dtype=torch.uint8, device=self.device)
            probe.copy_(pt[:16])
            self.peer_ptrs.append(pt.data_ptr())

    # ------------------------------------------------------------------ helpers
    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        esz = torch.empty(0, dtype=dtype).element_size()
        return self.local[offset: offset + n * esz].view(dtype).view(*shape)

    def peer_addr(self, rank: int, offset: int) -> int:
        return self.peer_ptrs[rank] + offset

    def barrier(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
