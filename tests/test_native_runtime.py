"""Native C++ runtime: arena / bump allocators, memory helpers, and the CPU oracles against the PyTorch restatements
(reference: cpp/tests/test_router_dispatch.cpp, tests/test_buffer_pool.py, test_heap_allocator.py, test_expert_cache.py,
test_cpu_dequant.py, test_logits_ops.py)."""
import pytest
import torch

from metal_marlin_b200 import ref
from metal_marlin_b200.formats import fp4 as fp4fmt
from metal_marlin_b200.memory import (Arena, BumpAllocator, ExpertCache, MemoryPressureMonitor, PinnedPool, PressureLevel, WeightStreamer,
                                      WorkspaceBuffer)
from metal_marlin_b200.ops import reference as pyref


def test_arena_best_fit_coalesce_pin_evict():
    a = Arena(4096, alignment=256)
    x = a.alloc((256,), torch.float32, tag="x")             # 1024 B
    y = a.alloc((512,), torch.bfloat16, tag="y")            # 1024 B
    z = a.alloc((1024,), torch.uint8, tag="z")
    assert a.offset_of(x) == 0 and a.offset_of(y) == 1024 and a.offset_of(z) == 2048
    x.fill_(3.0)
    assert float(a.slab[:1024].view(torch.float32).sum()) == 3.0 * 256
    a.free(y)
    small = a.alloc((100,), torch.uint8)                    # best fit: the 1024-byte hole, not the tail
    assert a.offset_of(small) == 1024
    a.free(small), a.free(x)
    assert a.stats()["largest_free"] == 2048                # holes coalesced
    with pytest.raises(MemoryError):
        a.alloc((4096,), torch.uint8)
    evicted = []
    a.on_evict = lambda off, tag: evicted.append(tag)
    a.pin(z)
    w = a.alloc((1024,), torch.uint8, priority=0, tag="w")  # offsets 0..1023
    with pytest.raises(MemoryError):
        a.alloc((4096,), torch.uint8, priority=5, allow_evict=True)          # z is pinned: cannot make room
    a.pin(z, False)
    big = a.alloc((4096,), torch.uint8, priority=5, allow_evict=True)
    assert sorted(evicted) == ["w", "z"] and a.offset_of(big) == 0 and a.stats()["evictions"] >= 2
    a.close()


def test_bump_allocator_and_workspace():
    b = BumpAllocator(4096, alignment=128)
    t1 = b.alloc((10,), torch.float32)
    m = b.mark()
    t2 = b.alloc((100,), torch.bfloat16)
    assert t2.data_ptr() - t1.data_ptr() == 128
    b.release(m)
    assert b.alloc((1,), torch.uint8).data_ptr() == t2.data_ptr()
    b.reset()
    assert b.cursor == 0 and b.high_water >= 328
    with pytest.raises(MemoryError):
        b.alloc((5000,), torch.uint8)
    ws = WorkspaceBuffer()
    p = ws.get("partials", (4, 8), torch.float32)
    assert ws.get("partials", (2, 8), torch.float32).data_ptr() == p.data_ptr() and ws.nbytes() == 128


def test_streaming_expert_cache_pressure():
    pool = PinnedPool()
    buf = pool.get(5000)
    assert buf.numel() == 8192
    pool.put(buf)
    assert pool.get(6000).data_ptr() == buf.data_ptr() and pool.hits == 1
    layers = [{"w": torch.full((4, 4), float(i))} for i in range(5)]
    got = [float(d["w"].sum()) for d in WeightStreamer("cpu", depth=2).stream_layers(layers)]
    assert got == [16.0 * i for i in range(5)]
    loads = []
    cache = ExpertCache(2, lambda k: loads.append(k) or f"expert{k}")
    for k in [(0, 1), (0, 2), (0, 1), (0, 3), (0, 2)]:
        cache.get(k)
    assert loads == [(0, 1), (0, 2), (0, 3), (0, 2)] and cache.hits == 1 and cache.evictions == 2 and cache.hot_keys(1)[0] in [(0, 1), (0, 2)]
    state = {"free": 50}
    events = []
    mon = MemoryPressureMonitor(probe=lambda: (state["free"], 100))
    mon.register(lambda lvl, used: events.append(lvl))
    assert mon.check() == PressureLevel.NORMAL
    state["free"] = 10
    assert mon.check() == PressureLevel.WARNING
    state["free"] = 2
    assert mon.check() == PressureLevel.CRITICAL and events == [PressureLevel.WARNING, PressureLevel.CRITICAL]


def test_cpu_oracles_agree_with_pytorch_restatements():
    torch.manual_seed(0)
    w = torch.randn(24, 128) * 0.1
    codes, scales = fp4fmt.quantize_codes(w, 32)
    torch.testing.assert_close(ref.dequant_fp4(codes, scales), fp4fmt.dequantize_codes(codes, scales), rtol=0, atol=0)
    x = (torch.randn(5, 64) * 0.5).to(torch.bfloat16)
    rw = torch.randn(16, 64).to(torch.bfloat16)
    bias = torch.randn(16) * 0.1
    for scoring in (0, 1):
        ids, wts = ref.router_topk(x, rw, bias if scoring else None, topk=4, scoring=scoring, renorm=True, routed_scale=1.5)
        ids2, wts2, _ = pyref.moe_router(x, rw, bias=bias if scoring else None, topk=4, scoring=scoring, renorm=True, routed_scale=1.5)
        assert torch.equal(ids.sort(1).values, ids2.sort(1).values)
        torch.testing.assert_close(wts.sort(1).values, wts2.sort(1).values, rtol=1e-4, atol=1e-5)
    lg = torch.randn(3, 50) * 3
    p = ref.logits_process(lg, temperature=0.7, top_k=10, top_p=0.9)
    assert torch.allclose(p.sum(1), torch.ones(3), atol=1e-5) and int((p > 0).sum(1).max()) <= 10
    assert torch.equal(ref.logits_process(lg, temperature=0.0).argmax(1), lg.argmax(1))
    hist = lg.argmax(1, keepdim=True)
    p_pen = ref.logits_process(lg, temperature=1.0, rep_penalty=5.0, history=hist)
    p_raw = ref.logits_process(lg, temperature=1.0)
    assert (p_pen.gather(1, hist) < p_raw.gather(1, hist)).all()
    ids = torch.tensor([[2, 0], [1, 2], [-1, 0]])
    order, offsets, counts = ref.group_tokens(ids, 3)
    assert counts.tolist() == [2, 1, 2] and offsets.tolist() == [0, 2, 3, 5] and order.tolist() == [1, 5, 2, 0, 3]
    plan = ref.plan_grouped_gemm(torch.tensor([70, 0, 10, 5]), torch.tensor([0, 70, 70, 80, 85]), torch.tensor([4, 4, 2, 4]), 64)
    assert plan.tolist() == [[0, 2, 2, 70, 10], [1, 4, 0, 0, 64], [1, 4, 0, 64, 6], [1, 4, 3, 80, 5]]
    pruned, mask = ref.prune_2_4(torch.tensor([[1.0, -3.0, 0.5, 2.0, 4.0, 4.0, -5.0, 0.1]]))
    assert pruned.tolist() == [[0.0, -3.0, 0.0, 2.0, 4.0, 0.0, -5.0, 0.0]] and int(mask.sum()) == 4
