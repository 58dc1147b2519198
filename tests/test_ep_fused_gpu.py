"""Expert-parallel prefill with the token exchange inside our kernels (``csrc/ep_comm.cu``): dispatch by peer stores, tile
list built on the device after the senders' flags, down-projection epilogue storing into the token owners' buffers.

* One GPU: all ranks' buffers live on the same device and the ranks are stepped phase by phase (every dispatch, then every
  expert pass, then every combine), so no launch ever waits for a later one.
* Two GPUs: one child process per GPU over real peer memory (NVLS off, plain peer stores), against the NCCL all-to-all
  path and the unsharded layer.
"""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _banks(E, ns, H, I, gs):
    from metal_marlin_b200.ops.weights import FP4ExpertBank
    gu = FP4ExpertBank.from_float(torch.randn(E + ns, 2 * I, H, device=DEV) * 0.05, gs)
    dn = FP4ExpertBank.from_float(torch.randn(E + ns, H, I, device=DEV) * 0.05, gs)
    return gu, dn


@pytest.mark.parametrize("ep,T,E,topk,H,I,gs,skew", [(2, 48, 8, 2, 256, 128, 64, False), (4, 40, 16, 4, 512, 192, 64, True),
                                                     (2, 300, 64, 4, 2048, 512, 128, True)])
def test_fused_dispatch_gemm_combine_emulated_ranks(ep, T, E, topk, H, I, gs, skew):
    from metal_marlin_b200 import ops
    from metal_marlin_b200.parallel.ep import EPExchange, ExpertParallelMoE
    torch.manual_seed(ep * 100 + T)
    gu, dn = _banks(E, 0, H, I, gs)
    nw = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16)
    # ranks hold different numbers of tokens (the last one none at all when skewed)
    per = [T] * ep
    if skew:
        per = [T, T // 3] + [T // 2] * (ep - 3) + [0] if ep > 2 else [T, T // 3]
    xs, idss, wtss, adds = [], [], [], []
    for r in range(ep):
        n = per[r]
        xs.append(torch.randn(n, H, device=DEV).to(torch.bfloat16))
        ids = torch.stack([torch.randperm(E, device=DEV)[:topk] for _ in range(n)]).to(torch.int32) if n else \
            torch.zeros(0, topk, dtype=torch.int32, device=DEV)
        if skew and n:
            ids[: n // 2, 0] = 0          # one hot expert; the other slots stay distinct from it
            ids[: n // 2, 1:] = torch.stack([1 + torch.randperm(E - 1, device=DEV)[: topk - 1] for _ in range(n // 2)]).to(torch.int32)
            ids[-1, -1] = -1              # a dropped pair
        idss.append(ids)
        wtss.append(torch.rand(n, topk, device=DEV))
        adds.append(torch.randn(n, H, device=DEV).to(torch.bfloat16))
    exs = EPExchange.emulated(ep, H, max(per), topk, DEV)
    moes = [ExpertParallelMoE(gu, dn, E, 0, r, ep) for r in range(ep)]
    for rep in range(2):          # twice: the buffers, counters and flags are reused from step to step
        states = [moes[r].fused_dispatch(exs[r], xs[r], idss[r], wtss[r], norm_w=nw) for r in range(ep)]
        for r in range(ep):
            moes[r].fused_experts(exs[r], expected_rows=sum(per) * topk // ep)
        outs = [moes[r].fused_combine(exs[r], states[r], add0=adds[r]) for r in range(ep)]
        torch.cuda.synchronize()
        assert ops.check_status(torch.device(DEV)) == 0
        for r in range(ep):
            assert exs[r].check() == 0
            if per[r] == 0:
                continue
            with ops.force_reference():
                ref = ops.moe_forward(xs[r], gu, dn, idss[r], wtss[r], norm_w=nw, out_add=adds[r]).float()
            err = float((outs[r].float() - ref).abs().max() / ref.abs().max())
            assert err < 4e-2, (rep, r, err)


_CHILD = r"""
import os, sys, json, torch, torch.distributed as dist
sys.path.insert(0, os.environ["MMB_REPO"])
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
from metal_marlin_b200 import ops
from metal_marlin_b200.ops.weights import FP4ExpertBank
from metal_marlin_b200.parallel.ep import EPExchange, ExpertParallelMoE
E, topk, H, I, gs, T = 16, 4, 512, 256, 64, 96 + 8 * rank
torch.manual_seed(7)                       # same banks on every rank
gu = FP4ExpertBank.from_float(torch.randn(E, 2 * I, H, device=dev) * 0.05, gs)
dn = FP4ExpertBank.from_float(torch.randn(E, H, I, device=dev) * 0.05, gs)
nw = (1 + 0.1 * torch.randn(H, device=dev)).to(torch.bfloat16)
torch.manual_seed(100 + rank)              # different tokens
x = torch.randn(T, H, device=dev).to(torch.bfloat16)
ids = torch.stack([torch.randperm(E, device=dev)[:topk] for _ in range(T)]).to(torch.int32)
wts = torch.rand(T, topk, device=dev)
add = torch.randn(T, H, device=dev).to(torch.bfloat16)
moe = ExpertParallelMoE(gu, dn, E, 0, rank, world)
ex = EPExchange.create(H, 160, topk, dev)
errs = []
for rep in range(3):
    out = moe.forward_fused(ex, x, ids, wts, norm_w=nw, add0=add)
    base = moe.forward_dispatch(x, ids, wts, norm_w=nw).float() + add.float()
    with ops.force_reference():
        ref = ops.moe_forward(x, gu, dn, ids, wts, norm_w=nw, out_add=add).float()
    errs.append([float((out.float() - ref).abs().max() / ref.abs().max()), float((base - ref).abs().max() / ref.abs().max())])
# the same exchange over trellis experts (mixed 2-8 bits, codes decoded inside the grouped tensor-core GEMMs)
from metal_marlin_b200.layers import TrellisLinear
from metal_marlin_b200.ops import generic
from metal_marlin_b200.parallel.ep import GenericExpertParallelMoE
bits = [2, 3, 4, 5, 6, 8]
tg, td = [], []
for e in range(E):
    b = bits[e % len(bits)]
    tg.append(generic.CatWeight([TrellisLinear.random(I, H, b, 64, dev, seed=3 * e, std=0.05), TrellisLinear.random(I, H, b, 64, dev, seed=3 * e + 1, std=0.05)]))
    td.append(TrellisLinear.random(H, I, b, 64, dev, seed=3 * e + 2, std=0.05))
tbank = generic.GenericExpertBank(tg, td)
tmoe = GenericExpertParallelMoE(tbank, E, rank, world)
out_t = tmoe.forward_fused(ex, x, ids, wts, norm_w=nw, add0=add)
ref_t = generic.moe_forward(x, tbank, ids, wts, norm_w=nw, out_add=add).float()
trellis_err = float((out_t.float() - ref_t).abs().max() / ref_t.abs().max())
torch.cuda.synchronize()
res = {"rank": rank, "errs": errs, "trellis_err": trellis_err, "status": ex.check(), "gemm_status": ops.check_status(dev)}
print("RESULT " + json.dumps(res), flush=True)
dist.barrier()
dist.destroy_process_group()
"""


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_expert_parallel_multi_gpu(world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = _free_port()
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    procs = []
    for r in range(world):
        env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r),
                   MMB_REPO=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    from conftest import collect_children
    outs = collect_children(procs, 240)
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{o[-3000:]}"
        res = json.loads([l for l in o.splitlines() if l.startswith("RESULT ")][-1][7:])
        assert res["status"] == 0 and res["gemm_status"] == 0, res
        for fused_err, nccl_err in res["errs"]:
            assert fused_err < 4e-2 and nccl_err < 4e-2, res
        assert res["trellis_err"] < 4e-2, res
