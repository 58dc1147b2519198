"""Symmetric memory on this library's own allocator (``csrc/symm_vmm.cpp``): every rank creates an exportable physical
allocation on its GPU, the file descriptors travel to the peers over Unix-domain sockets (``SCM_RIGHTS``), every rank maps
every peer's allocation into its address space - after which kernels store into and load from peer memory with plain
pointers - and, where asked, all copies are bound to one NVSwitch multicast object whose mapping serves ``multimem``
instructions.

Rendezvous: socket paths are derived from a job tag agreed through the process group (an object broadcast); rank ``r`` listens
on ``<dir>/mmb200-<tag>-<r>.sock`` and serves its descriptor to every peer that connects.  Nothing here launches a kernel or
waits on the device; all blocking calls are socket operations with timeouts.
"""
from __future__ import annotations

import os
import socket
import tempfile
import threading
import uuid
from typing import List, Optional

import torch
import torch.distributed as dist

SOCKET_TIMEOUT_S = 60.0


def _ops():
    from .. import _build
    _build.load()
    return torch.ops.mmb200


def available() -> int:
    """0: driver API not reachable; 1: exportable allocations; 2: also multicast objects."""
    try:
        return int(_ops().vmm_available())
    except Exception:
        return 0


def _check(v: int, what: str) -> int:
    if v <= 0:
        raise RuntimeError(f"{what} failed (driver error {-v})")
    return v


class _FdServer:
    """Hands one file descriptor to every peer that connects (``n`` connections, then stops)."""

    def __init__(self, path: str, fds: List[int], n: int):
        self.path, self.fds, self.n = path, fds, n
        self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        if os.path.exists(path):
            os.unlink(path)
        self.sock.bind(path)
        self.sock.listen(max(1, n))
        self.sock.settimeout(SOCKET_TIMEOUT_S)
        self.error: Optional[BaseException] = None
        self.thread = threading.Thread(target=self._serve, daemon=True)
        self.thread.start()

    def _serve(self):
        try:
            for _ in range(self.n):
                conn, _ = self.sock.accept()
                with conn:
                    conn.settimeout(SOCKET_TIMEOUT_S)
                    socket.send_fds(conn, [b"fd"], self.fds)
        except BaseException as e:      # reported by join()
            self.error = e
        finally:
            self.sock.close()
            try:
                os.unlink(self.path)
            except OSError:
                pass

    def join(self):
        self.thread.join(SOCKET_TIMEOUT_S + 5)
        if self.error is not None:
            raise RuntimeError(f"descriptor exchange failed: {self.error!r}")


def _fetch_fds(path: str, count: int) -> List[int]:
    import time
    deadline = time.monotonic() + SOCKET_TIMEOUT_S
    while True:
        try:
            s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            s.settimeout(SOCKET_TIMEOUT_S)
            s.connect(path)
            break
        except (FileNotFoundError, ConnectionRefusedError):
            s.close()
            if time.monotonic() > deadline:
                raise TimeoutError(f"no peer is listening on {path}")
            time.sleep(0.01)
    with s:
        _, fds, _, _ = socket.recv_fds(s, 16, count)
    if len(fds) != count:
        raise RuntimeError(f"expected {count} descriptor(s) from {path}, got {len(fds)}")
    return list(fds)


class VmmExchange:
    """``nbytes`` on every rank of ``group`` (rounded up to the allocation granularity), all peers' copies mapped locally.

    ``local``: uint8 tensor over this rank's copy; ``peer_ptrs[r]``: device address of rank r's copy in THIS process;
    ``multicast_ptr``: the ``multimem`` address of all copies (0 without multicast)."""

    def __init__(self, nbytes: int, device, group=None, multicast: bool = False, socket_dir: Optional[str] = None):
        K = _ops()
        if available() < 1:
            raise RuntimeError("the CUDA virtual-memory API is not reachable through this driver")
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.device = torch.device(device)
        dev = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.dev = dev
        tag = [uuid.uuid4().hex[:12] if self.rank == 0 else None]
        dist.broadcast_object_list(tag, src=dist.get_global_rank(self.group, 0) if hasattr(dist, "get_global_rank") else 0, group=self.group)
        sdir = socket_dir or os.environ.get("MMB200_SOCKET_DIR") or tempfile.gettempdir()
        path = lambda r, kind="mem": os.path.join(sdir, f"mmb200-{tag[0]}-{kind}-{r}.sock")
        self._ids: List[int] = []
        self._peer_ids = {}
        devs = [None] * self.world
        dist.all_gather_object(devs, dev, group=self.group)
        self.peer_devices = [int(d) for d in devs]          # device ordinal each rank's copy physically lives on
        self.mem_id = _check(int(K.vmm_create(dev, int(nbytes))), "cuMemCreate / map")
        self.nbytes = int(K.vmm_size(self.mem_id))
        fd = _check(int(K.vmm_export_fd(self.mem_id)) + 1, "cuMemExportToShareableHandle") - 1
        server = _FdServer(path(self.rank), [fd], self.world - 1)
        self.peer_ptrs: List[int] = [0] * self.world
        self.peer_ptrs[self.rank] = int(K.vmm_ptr(self.mem_id))
        try:
            for off in range(1, self.world):
                r = (self.rank + off) % self.world
                (pfd,) = _fetch_fds(path(r), 1)
                try:
                    pid = _check(int(K.vmm_import_fd(pfd, self.nbytes, dev)), f"import of rank {r}'s allocation")
                finally:
                    os.close(pfd)
                self._ids.append(pid)
                self._peer_ids[r] = pid
                self.peer_ptrs[r] = int(K.vmm_ptr(pid))
            server.join()
        finally:
            K.vmm_close_fd(fd)
        self.local = K.vmm_tensor(self.mem_id, self.nbytes, dev)
        self.multicast_ptr = 0
        self.mc_id = 0
        if multicast and self.world > 1 and available() >= 2:
            self._init_multicast(path)
        dist.barrier(self.group)
        import atexit
        import weakref
        ref = weakref.ref(self)
        atexit.register(lambda: ref() is not None and ref()._release())

    def _agree(self, ok: bool) -> bool:
        """True when every rank reports success (all ranks take the same branch afterwards)."""
        flags = [None] * self.world
        dist.all_gather_object(flags, bool(ok), group=self.group)
        return all(flags)

    def _init_multicast(self, path) -> None:
        """Binds all copies to one NVSwitch multicast object.  Every stage is agreed between the ranks; if any rank fails a
        stage all ranks give the object up together and continue with peer pointers only (``multicast_ptr`` stays 0)."""
        K = _ops()
        server, mfd = None, -1
        ok = True
        if self.rank == 0:
            self.mc_id = int(K.mc_create(self.world, self.nbytes))
            ok = self.mc_id > 0
            if ok:
                mfd = int(K.mc_export_fd(self.mc_id))
                ok = mfd >= 0
        if not self._agree(ok):                     # the fabric / driver has no multicast: nobody waits for a descriptor
            self._drop_multicast(mfd)
            return
        try:
            if self.rank == 0:
                server = _FdServer(path(0, "mc"), [mfd], self.world - 1)
            else:
                (pfd,) = _fetch_fds(path(0, "mc"), 1)
                try:
                    self.mc_id = int(K.mc_import_fd(pfd, self.world, self.nbytes))
                finally:
                    os.close(pfd)
                ok = self.mc_id > 0
            if ok:
                ok = int(K.mc_add_device(self.mc_id, self.dev)) == 0
            if server is not None:
                server.join()
        except Exception:
            ok = False
        if not self._agree(ok):
            self._drop_multicast(mfd)
            return
        if self.rank == 0:
            K.vmm_close_fd(mfd)
            mfd = -1
        ok = int(K.mc_bind(self.mc_id, self.mem_id)) == 0          # every device is part of the object (agreed above)
        self._bound = ok
        if not self._agree(ok):
            self._drop_multicast(mfd)
            return
        self.multicast_ptr = int(K.mc_map(self.mc_id, self.dev))
        if not self._agree(self.multicast_ptr != 0):
            self.multicast_ptr = 0
            self._drop_multicast(mfd)

    def _drop_multicast(self, mfd: int = -1) -> None:
        K = _ops()
        if mfd >= 0:
            K.vmm_close_fd(mfd)
        if self.mc_id > 0:
            if getattr(self, "_bound", False):
                K.mc_unbind(self.mc_id, self.dev, self.mem_id)
            K.vmm_free(self.mc_id)
        self.mc_id = 0
        self._bound = False
        self.multicast_ptr = 0

    def read_peer(self, r: int, offset: int, out: torch.Tensor) -> torch.Tensor:
        """Copy ``out.numel() * out.element_size()`` bytes at ``offset`` of rank ``r``'s copy into the local tensor ``out``
        (a device-to-device copy issued on this rank's device, through the mapping made for it)."""
        n = out.numel() * out.element_size()
        assert out.is_contiguous() and 0 <= offset and offset + n <= self.nbytes
        _ops().vmm_copy(out.data_ptr(), self.peer_ptrs[r] + offset, n, self.dev)
        return out

    def write_peer(self, r: int, offset: int, src: torch.Tensor) -> None:
        """Copy the local tensor ``src`` to ``offset`` of rank ``r``'s copy (stores into peer memory)."""
        n = src.numel() * src.element_size()
        assert src.is_contiguous() and 0 <= offset and offset + n <= self.nbytes
        _ops().vmm_copy(self.peer_ptrs[r] + offset, src.data_ptr(), n, self.dev)

    def _release(self) -> None:
        """Local teardown (no communication): unbind from the multicast object, unmap the peers' copies, free the own copy.
        Also runs at interpreter exit, so that a process never leaves with its memory still bound to a multicast object."""
        K = _ops()
        try:
            torch.cuda.synchronize(self.device)
        except Exception:
            pass
        self.local = None
        self._drop_multicast()
        for i in self._ids:
            K.vmm_free(i)
        self._ids = []
        if self.mem_id:
            K.vmm_free(self.mem_id)
            self.mem_id = 0

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)                   # nobody still stores into a copy that is about to be unmapped
        self._release()
        dist.barrier(self.group)
