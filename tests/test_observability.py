"""Tracing, launch tracing, roofline arithmetic, NaN guard and checkpoint utilities (reference: tests/test_tracing.py,
test_launch_tracing.py, test_roofline.py, test_nan_guard.py, test_checkpoint.py)."""
import json

import torch

from metal_marlin_b200 import ops
from metal_marlin_b200.models.config import get_preset
from metal_marlin_b200.profiling import (KernelTimer, RooflinePoint, decode_step_cost, fused_collective_roof_seconds, gemm_flops, load_peaks,
                                         tracing)
from metal_marlin_b200.utils import (LazyCheckpoint, NaNGuard, filter_weights, load_checkpoint, remap_weight_keys, save_checkpoint)


def test_chrome_trace_and_launch_tracer(tmp_path):
    tracing.enable(True, True)
    tracing.clear()
    try:
        with tracing.trace_scope("prefill", tokens=16):
            with tracing.trace_scope("layer0", cat="layer"):
                pass
        tracing.record_event("manual", 1.0, 2.0)
        n = tracing.write_trace(str(tmp_path / "t.json"))
        ev = json.load(open(tmp_path / "t.json"))["traceEvents"]
        assert n == 3 and {e["name"] for e in ev} == {"prefill", "layer0", "manual"}
        assert all(e["ph"] == "X" and e["dur"] >= 0 for e in ev) and ev[-1]["args"] == {}
        lt = tracing.LaunchTracer()
        with lt.trace_region("step"):
            lt.record_kernel("gemv", 3)
            lt.record_copy("h2d", 8)
            lt.record_wait()
            lt.record_commit()
        assert lt.regions["step"]["kernel:gemv"] == 3 and lt.counters["bytes_h2d"] == 8 and lt.counters["waits"] == 1
        lt.write_json(str(tmp_path / "l.json"))
        assert json.load(open(tmp_path / "l.json"))["regions"]["step"]["graph_replays"] == 1
    finally:
        tracing.enable(False, False)
    tracing.clear()
    with tracing.trace_scope("off"):
        pass
    assert tracing.write_trace(str(tmp_path / "t2.json")) == 0


def test_roofline_points_and_decode_cost():
    peaks = load_peaks()
    assert peaks["hbm_gbs"] > 1000 and peaks["source"] in ("measured", "fallback")
    gemv = RooflinePoint("gemv", gemm_flops(1, 4096, 4096), 4096 * 4096 / 2, 2e-6, peaks)
    assert gemv.bound == "memory" and 0 < gemv.fraction_of_roof < 2
    gemm = RooflinePoint("gemm", gemm_flops(8192, 8192, 8192), 3 * 8192 * 8192 * 2, 1e-3, peaks)
    assert gemm.bound == "compute" and abs(gemm.achieved_tflops - 1099.5) < 1 and gemm.row()["of"] == peaks["source"]
    c = decode_step_cost(get_preset("glm-4.7-flash"), batch=1, ctx=4096)
    assert 1e9 < c["weight_bytes"] < 4e9 and c["kv_bytes"] == 4096 * 576 * 2 * 47
    t = fused_collective_roof_seconds(flops=1e12, nvlink_bytes=1e9, peaks=peaks)
    assert abs(t - 1e9 / 770e9) < 1e-6
    timer = KernelTimer(warmup=1, iters=3, flush_l2=False)
    assert timer.time(lambda: torch.ones(10).sum(), "sum") > 0 and "sum" in timer.records


def test_nan_guard_and_checkpoint_utils(tmp_path):
    g = NaNGuard()
    good, bad = torch.ones(3), torch.tensor([1.0, float("nan"), 2.0])
    assert torch.equal(g.run(lambda: good), good)
    assert torch.equal(g.run(lambda: bad, lambda: good), good) and g.stats.fallbacks == 1
    assert torch.equal(g.run(lambda: bad), torch.tensor([1.0, 0.0, 2.0])) and g.stats.unrecovered == 1 and g.stats.nan_detected == 2
    sd = {f"model.layers.{i}.w": torch.full((4,), float(i)) for i in range(4)}
    sd["lm_head.weight"] = torch.ones(2, 2)
    files = save_checkpoint(sd, str(tmp_path / "sh"), shard_bytes=32)
    assert len(files) >= 2
    back = load_checkpoint(str(tmp_path / "sh"))
    assert set(back) == set(sd) and float(back["model.layers.3.w"][0]) == 3.0
    assert set(load_checkpoint(str(tmp_path / "sh"), keys=["lm_head.weight"])) == {"lm_head.weight"}
    lazy = LazyCheckpoint(str(tmp_path / "sh"))
    assert len(lazy) == 5 and lazy.reads == 0 and float(lazy["model.layers.2.w"][0]) == 2.0 and lazy.reads == 1
    rem = remap_weight_keys(sd, {r"^model\.": "model.language_model."})
    assert "model.language_model.layers.0.w" in rem and "lm_head.weight" in rem
    assert set(filter_weights(sd, include=r"layers\.[01]\.")) == {"model.layers.0.w", "model.layers.1.w"}
    assert "lm_head.weight" not in filter_weights(sd, exclude="lm_head")


def test_server_monitor_parses_and_renders_metrics():
    from metal_marlin_b200.serving import monitor as mon
    text = """# HELP metal_marlin_requests_total Total requests
# TYPE metal_marlin_requests_total counter
metal_marlin_requests_total 12
metal_marlin_active_requests 3
metal_marlin_latency_ms{quantile="0.5"} 41.5
metal_marlin_latency_ms{quantile="0.95"} 90.25
metal_marlin_latency_ms{quantile="0.99"} 120
metal_marlin_tokens_total{type="prompt"} 1000
metal_marlin_tokens_total{type="completion"} 400
metal_marlin_queue_depth 2
metal_marlin_gpu_memory_mb 20480.0
metal_marlin_throughput_tok_sec 133.700
moe_tokens_processed_total 5000
garbage line
"""
    m = mon.parse_metrics(text)
    assert m["metal_marlin_requests_total"] == 12 and m['metal_marlin_latency_ms{quantile="0.95"}'] == 90.25 and len(m) == 11
    later = dict(m)
    later["metal_marlin_requests_total"] = 16
    later['metal_marlin_tokens_total{type="completion"}'] = 700
    table = mon.render(later, m, 2.0, {"status": "ok"})
    assert "status" in table and "ok" in table and "16 / 3" in table and "1000 / 700" in table
    assert "41.5 / 90.2 / 120.0" in table and "2.00" in table and "150.0" in table and "5000 / 0" in table
    lines = []
    rc = mon.run("http://x", once=True, out=lines.append, fetch_fn=lambda url: (m, {"status": "ok"}))
    assert rc == 0 and len(lines) == 1 and "requests total / active" in lines[0]

    def failing(url):
        raise OSError("connection refused")
    assert mon.run("http://x", once=True, out=lines.append, fetch_fn=failing) == 1 and "connection refused" in lines[-1]
    assert mon.run("http://x", interval=0.0, polls=2, out=lines.append, fetch_fn=lambda url: (later, {})) == 0
