"""Rank-failure detection on CPU processes: a rank that leaves between steps, a rank that goes silent, and the
device-status path of the step guard with a fake exchange context.  Failures are made on the host only."""
import os
import socket
import time
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from metal_marlin_b200.parallel.health import Heartbeat, PeerFailure, StepGuard


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, mode, q):
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=timedelta(seconds=30))
    hb = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=0.6).start()
    guard = StepGuard(hb)
    steps, err = 0, None
    store.add("ready", 1)                       # start together: process start-up times differ by seconds
    while int(store.add("ready", 0)) < world:
        time.sleep(0.01)
    try:
        for i in range(200):
            if rank == 1 and i == 3:
                if mode == "leave":
                    hb.leave()                  # orderly: between steps, nothing in flight
                else:
                    hb.stop()                   # silent: the heartbeat thread dies, the process lingers
                    time.sleep(3.0)
                break
            guard.run(lambda: time.sleep(0.02))
            steps += 1
    except PeerFailure as e:
        err = (e.ranks, e.reason)
    q.put((rank, steps, err))
    if rank == 0:
        time.sleep(0.5)                         # keep the store alive until the others reported
    hb.stop()


@pytest.mark.parametrize("mode", ["leave", "silent"])
def test_survivors_detect_a_lost_rank_before_the_next_step(mode):
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        r, steps, err = q.get(timeout=60)
        res[r] = (steps, err)
    for p in procs:
        p.join(timeout=30)
    assert res[1] == (3, None)
    for r in (0, 2):
        steps, err = res[r]
        assert err is not None and err[0] == [1], res
        assert 2 <= steps < 200
        assert ("left the job" in err[1]) if mode == "leave" else ("no heartbeat" in err[1])


def test_step_guard_reports_device_wait_expiry():
    class FakeStore(dict):
        def set(self, k, v):
            self[k] = v.encode() if isinstance(v, str) else v

        def get(self, k):
            return self[k]

    class FakeCtx:
        code = 0

        def check(self):
            return self.code

    store = FakeStore()
    hb = Heartbeat(store, 0, 1)
    ctx = FakeCtx()
    guard = StepGuard(hb, ctx)
    assert guard.run(lambda: 7) == 7
    ctx.code = 101                              # the bounded wait on source rank 1 expired
    with pytest.raises(PeerFailure) as e:
        guard.run(lambda: 7)
    assert e.value.ranks == [1] and "status 101" in str(e.value)


def test_status_codes_are_decoded_by_range():
    """Only three code ranges name a peer; everything else is a local wait or the capacity overflow."""
    from metal_marlin_b200.parallel.health import (DeviceWaitExpired, ExpertCapacityOverflow, decode_status,
                                                   raise_for_status)
    assert decode_status(0)[0] == "ok"
    assert decode_status(103)[:2] == ("peer", [3])
    assert decode_status(121)[:2] == ("peer", [0]) and decode_status(128)[:2] == ("peer", [7])
    assert decode_status(145)[:2] == ("peer", [5])
    for code in (1, 2, 3, 4, 42, 110, 200, 999):
        assert decode_status(code)[:2] == ("local", []), code
        with pytest.raises(DeviceWaitExpired):
            raise_for_status(code)
    assert decode_status(120)[0] == "capacity"
    with pytest.raises(ExpertCapacityOverflow):
        raise_for_status(120)
    with pytest.raises(PeerFailure) as e:
        raise_for_status(142)
    assert e.value.ranks == [2]
    raise_for_status(0)


def test_step_guard_keeps_non_peer_codes_apart():
    from metal_marlin_b200.parallel.health import DeviceWaitExpired, ExpertCapacityOverflow

    class FakeStore(dict):
        def set(self, k, v):
            self[k] = v.encode() if isinstance(v, str) else v

        def get(self, k):
            return self[k]

    class FakeCtx:
        code = 0

        def check(self):
            return self.code

    ctx = FakeCtx()
    guard = StepGuard(Heartbeat(FakeStore(), 0, 1), ctx)
    for code, exc in ((110, DeviceWaitExpired), (200, DeviceWaitExpired), (120, ExpertCapacityOverflow)):
        ctx.code = code
        with pytest.raises(exc):
            guard.run(lambda: 1)
    ctx.code = 125
    with pytest.raises(PeerFailure) as e:
        guard.run(lambda: 1)
    assert e.value.ranks == [4]


@pytest.mark.gpu
def test_bounded_device_waits_run_out_and_report():
    """The allowed form of a device-side failure test: a flag that nothing sets.  The wait limit is taken from word 1 of
    the status array (microseconds), the kernels give up after it, leave their code in word 0 and return; the host turns
    the code into PeerFailure and the context stays usable.  No fault, no trap, no endless loop."""
    import time

    import torch
    from metal_marlin_b200 import ops
    from metal_marlin_b200.ops.weights import FP4ExpertBank
    from metal_marlin_b200.parallel.ep import EPExchange, ExpertParallelMoE
    from metal_marlin_b200.parallel.health import raise_for_status
    dev = torch.device("cuda", 0)
    assert ops.native_available()
    # ---- tensor-parallel consumer wait: two source flags, step 1, nobody publishes
    flags = torch.zeros(2, dtype=torch.int32, device=dev)
    step = torch.ones(1, dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    status[1] = 3000                                            # give up after 3 ms
    desc = torch.tensor([flags.data_ptr(), step.data_ptr(), status.data_ptr(), 2], dtype=torch.int64)
    t0 = time.perf_counter()
    ops.K.mmb200.tp_wait(desc)
    torch.cuda.synchronize(dev)
    assert time.perf_counter() - t0 < 0.5                        # far below the one-second default: the setting was honoured
    code = int(status[0])
    assert code in (100, 101), code

    class Ctx:
        def check(self):
            return code

    class Store(dict):
        def set(self, k, v):
            self[k] = v.encode() if isinstance(v, str) else v

        def get(self, k):
            return self[k]

    with pytest.raises(PeerFailure) as e:
        StepGuard(Heartbeat(Store(), 0, 1), Ctx()).run(lambda: None)
    assert e.value.ranks == [code - 100]
    # the wait returns at once when the flags are there
    status.zero_()
    flags.fill_(1)
    ops.K.mmb200.tp_wait(desc)
    torch.cuda.synchronize(dev)
    assert int(status[0]) == 0
    # ---- expert-parallel owner: rank 0 of two emulated ranks waits for senders that never dispatch
    E, H, I, topk = 4, 256, 128, 2
    torch.manual_seed(0)
    gu = FP4ExpertBank.from_float(torch.randn(E, 2 * I, H, device=dev) * 0.05, 64)
    dn = FP4ExpertBank.from_float(torch.randn(E, H, I, device=dev) * 0.05, 64)
    exs = EPExchange.emulated(2, H, 16, topk, dev)
    moe = ExpertParallelMoE(gu, dn, E, 0, 0, 2)
    exs[0].set_wait_limit_us(3000)
    exs[0].begin()
    t0 = time.perf_counter()
    moe.fused_experts(exs[0], expected_rows=16 * topk)
    torch.cuda.synchronize(dev)
    assert time.perf_counter() - t0 < 0.5
    code = exs[0].check()
    assert code in (121, 122), code
    with pytest.raises(PeerFailure) as e:
        raise_for_status(code)
    assert e.value.ranks == [code - 121]
    # the device is still usable
    assert float(torch.ones(8, device=dev).sum()) == 8.0 and ops.check_status(dev) == 0
