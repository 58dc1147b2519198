"""This library's own symmetric-memory allocator: descriptor exchange over Unix sockets (CPU), and allocation / export /
import / peer access on the GPU - two processes that map each other's allocation and exchange data through plain peer
pointers, stepped by host barriers (no kernel waits for another)."""
import os
import socket
import subprocess
import sys
import tempfile

import pytest
import torch

from metal_marlin_b200.parallel import vmm

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_descriptor_exchange_over_unix_sockets(tmp_path):
    r, w = os.pipe()
    path = str(tmp_path / "x.sock")
    srv = vmm._FdServer(path, [w], 2)
    got = [vmm._fetch_fds(path, 1)[0] for _ in range(2)]
    srv.join()
    os.write(got[0], b"hi")
    os.write(got[1], b"!!")
    assert os.read(r, 4) == b"hi!!"
    for fd in got + [r, w]:
        os.close(fd)
    assert not os.path.exists(path)
    with pytest.raises(TimeoutError):
        old, vmm.SOCKET_TIMEOUT_S = vmm.SOCKET_TIMEOUT_S, 0.05
        try:
            vmm._fetch_fds(str(tmp_path / "nobody.sock"), 1)
        finally:
            vmm.SOCKET_TIMEOUT_S = old


def test_availability_probe_is_safe_without_a_driver():
    assert vmm.available() in (0, 1, 2)


_CHILD = r"""
import os, sys, json, torch, torch.distributed as dist
sys.path.insert(0, os.environ["MMB_REPO"])
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
ndev = torch.cuda.device_count()
dev = torch.device("cuda", rank % ndev)
torch.cuda.set_device(dev)
dist.init_process_group("gloo")
from metal_marlin_b200.parallel.symm import SymmetricBuffer
from metal_marlin_b200.parallel import vmm
res = {"available": vmm.available()}
buf = SymmetricBuffer(3 << 20, dev)
res["backend"] = buf.backend
res["nbytes"] = buf.nbytes
assert buf.peer_ptrs[rank] == buf.local.data_ptr() and len(set(buf.peer_ptrs)) == world
# every rank writes its pattern into its own copy ...
buf.local.view(torch.int32)[: 1 << 18].copy_(torch.arange(1 << 18, dtype=torch.int32, device=dev) * (rank + 1))
buf.barrier()
# ... and reads the peers' copies through the mapped peer pointers (a device-to-device copy from the peer address)
ok = True
for r in range(world):
    view = buf._vmm.read_peer(r, 0, torch.empty(1 << 18, dtype=torch.int32, device=dev))      # copy out of the peer's copy
    ok = ok and bool(torch.equal(view, torch.arange(1 << 18, dtype=torch.int32, device=dev) * (r + 1)))
res["peer_reads"] = ok
buf.barrier()
# a peer store: rank r writes one word into its right neighbour's copy
nxt = (rank + 1) % world
buf._vmm.write_peer(nxt, 2 << 20, torch.tensor([1000 + rank], dtype=torch.int32, device=dev))
torch.cuda.synchronize()
buf.barrier()
res["peer_store"] = int(buf.local[2 << 20: (2 << 20) + 4].view(torch.int32)[0]) == 1000 + (rank - 1) % world
buf.close()
if rank == 0:
    print("RESULT " + json.dumps(res), flush=True)
dist.destroy_process_group()
"""


@pytest.mark.gpu
def test_two_processes_map_each_others_allocation(tmp_path):
    """Runs with one GPU (both processes on it) or more (one GPU per process)."""
    from conftest import collect_children
    world = 2
    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False, dir=str(tmp_path)) as f:
        f.write(_CHILD)
        script = f.name
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs = []
    for r in range(world):
        env = dict(os.environ, MMB_REPO=REPO, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   MMB200_SYMM_BACKEND="vmm", MMB200_SOCKET_DIR=str(tmp_path))
        procs.append(subprocess.Popen([sys.executable, script], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = collect_children(procs, 120)
    assert any(l.startswith("RESULT ") for l in outs[0].splitlines()), outs
    import json
    line = next(l for l in outs[0].splitlines() if l.startswith("RESULT "))
    res = json.loads(line[len("RESULT "):])
    assert res["available"] >= 1 and res["backend"] == "vmm" and res["nbytes"] >= 3 << 20
    assert res["peer_reads"] and res["peer_store"], res
