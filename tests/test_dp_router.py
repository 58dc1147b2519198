"""Data-parallel request router in front of two replica servers (mock model, CPU): requests reach both replicas, SSE streams
pass through unchanged, a dead replica is skipped, metrics are merged."""
import json
import os
import socket
import threading
import time

import pytest
import requests


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _serve(app, port):
    import uvicorn
    srv = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
    th = threading.Thread(target=srv.run, daemon=True)
    th.start()
    for _ in range(100):
        try:
            if requests.get(f"http://127.0.0.1:{port}/health", timeout=1).status_code == 200:
                break
        except Exception:
            time.sleep(0.1)
    return srv, th


@pytest.fixture(scope="module")
def cluster():
    os.environ["METAL_MARLIN_MOCK_MODEL"] = "1"
    os.environ["METAL_MARLIN_MOCK_MODEL_NAME"] = "mock-model"
    from metal_marlin_b200.serving import server as srv
    from metal_marlin_b200.serving.engine import EngineConfig
    from metal_marlin_b200.serving.router import ReplicaRouter, make_app
    srv.configure(EngineConfig(max_model_len=512, num_kv_blocks=128, request_timeout=30))
    # two listeners of the one in-process replica app stand in for two replicas; a third address has no listener
    p1, p2, dead, pr = _port(), _port(), _port(), _port()
    s1 = _serve(srv.app, p1)
    s2 = _serve(srv.app, p2)
    router = ReplicaRouter([f"http://127.0.0.1:{p1}", f"http://127.0.0.1:{p2}", f"http://127.0.0.1:{dead}"])
    sr = _serve(make_app(router), pr)
    yield f"http://127.0.0.1:{pr}", router
    for s, th in (sr, s1, s2):
        s.should_exit = True
        th.join(timeout=5)
    srv._engine.shutdown()
    os.environ.pop("METAL_MARLIN_MOCK_MODEL", None)


def test_router_spreads_requests_and_skips_dead_replica(cluster):
    base, router = cluster
    seen = set()
    for _ in range(6):
        r = requests.post(base + "/v1/completions", json={"model": "mock-model", "prompt": "hello", "max_tokens": 4, "temperature": 0})
        assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] == 4
        seen.add(r.headers["x-mmb200-replica"])
    assert seen == {"0", "1"}                       # both live replicas served; the dead one was tried at most once
    assert router.healthy == [True, True, False] or router.served[2] == 0
    h = requests.get(base + "/health").json()
    assert h["status"] == "ok" and h["replicas"]["healthy"][2] is False
    assert sum(router.inflight) == 0


def test_router_streams_sse_and_merges_metrics(cluster):
    base, router = cluster
    with requests.post(base + "/v1/chat/completions", stream=True,
                       json={"model": "mock-model", "stream": True, "max_tokens": 5, "temperature": 0,
                             "messages": [{"role": "user", "content": "hi"}]}) as r:
        assert r.status_code == 200 and r.headers["content-type"].startswith("text/event-stream")
        lines = [l.decode() for l in r.iter_lines() if l]
    assert lines[-1] == "data: [DONE]"
    first = json.loads(lines[0][6:])
    assert first["choices"][0]["delta"]["role"] == "assistant"
    m = requests.get(base + "/metrics").text
    assert 'mmb200_router_served{replica="0"}' in m and "# replica 1" in m
    assert requests.get(base + "/v1/models").json()["data"][0]["id"] == "mock-model"
    assert sum(router.inflight) == 0
