"""HTTP server against the mock model: routes, schemas, SSE framing, errors, metrics, concurrency.
Same approach as the reference's tests/test_openai_server.py (mock model behind METAL_MARLIN_MOCK_MODEL=1)."""
import json
import os
import socket
import threading
import time

import pytest
import requests


@pytest.fixture(scope="module")
def server():
    os.environ["METAL_MARLIN_MOCK_MODEL"] = "1"
    os.environ["METAL_MARLIN_MOCK_MODEL_NAME"] = "mock-model"
    import uvicorn
    from metal_marlin_b200.serving import server as srv
    from metal_marlin_b200.serving.engine import EngineConfig

    srv.configure(EngineConfig(max_model_len=512, num_kv_blocks=128, request_timeout=30))
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    userver = uvicorn.Server(uvicorn.Config(srv.app, host="127.0.0.1", port=port, log_level="warning"))
    th = threading.Thread(target=userver.run, daemon=True)
    th.start()
    base = f"http://127.0.0.1:{port}"
    for _ in range(100):
        try:
            if requests.get(base + "/health", timeout=1).status_code == 200:
                break
        except Exception:
            time.sleep(0.1)
    yield base
    userver.should_exit = True
    th.join(timeout=5)
    srv._engine.shutdown()
    os.environ.pop("METAL_MARLIN_MOCK_MODEL", None)


def test_health_and_models(server):
    h = requests.get(server + "/health").json()
    assert h["status"] == "ok" and h["model_loaded"] is True
    m = requests.get(server + "/v1/models").json()
    assert m["object"] == "list" and m["data"][0]["id"] == "mock-model" and m["data"][0]["owned_by"] == "metal-marlin"
    assert requests.get(server + "/v1/models/mock-model").status_code == 200
    r = requests.get(server + "/v1/models/nope")
    assert r.status_code == 404 and r.json()["error"]["code"] == "model_not_found"


def test_chat_completion(server):
    r = requests.post(server + "/v1/chat/completions", json={"model": "mock-model", "max_tokens": 8, "temperature": 0,
                                                              "messages": [{"role": "user", "content": "hi"}]})
    assert r.status_code == 200
    d = r.json()
    assert d["object"] == "chat.completion" and d["choices"][0]["message"]["role"] == "assistant"
    assert d["usage"]["completion_tokens"] == 8 and d["choices"][0]["finish_reason"] == "length"
    assert d["usage"]["total_tokens"] == d["usage"]["prompt_tokens"] + 8


def test_completion_n_and_echo(server):
    r = requests.post(server + "/v1/completions", json={"model": "mock-model", "prompt": "abc", "max_tokens": 4, "n": 2,
                                                         "temperature": 0, "echo": True})
    d = r.json()
    assert r.status_code == 200 and len(d["choices"]) == 2 and all(c["text"].startswith("abc") for c in d["choices"])
    assert d["choices"][0]["text"] == d["choices"][1]["text"]          # greedy -> identical samples


def test_streaming_sse_framing(server):
    r = requests.post(server + "/v1/chat/completions", stream=True,
                      json={"model": "mock-model", "max_tokens": 6, "temperature": 0, "stream": True,
                            "messages": [{"role": "user", "content": "stream please"}]})
    assert r.status_code == 200 and r.headers["content-type"].startswith("text/event-stream")
    lines = [l.decode() for l in r.iter_lines() if l]
    assert all(l.startswith("data: ") for l in lines) and lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    assert chunks[-1]["choices"][0]["finish_reason"] in ("stop", "length")
    assert all(c["object"] == "chat.completion.chunk" for c in chunks)


def test_validation_and_model_errors(server):
    assert requests.post(server + "/v1/chat/completions", json={"model": "mock-model", "messages": []}).status_code == 422
    r = requests.post(server + "/v1/chat/completions", json={"model": "other", "messages": [{"role": "user", "content": "x"}]})
    assert r.status_code == 404 and r.json()["error"]["type"] == "invalid_request_error"
    r = requests.post(server + "/v1/completions", json={"model": "mock-model", "prompt": "x" * 600, "max_tokens": 8})
    assert r.status_code == 400 and r.json()["error"]["code"] == "context_length_exceeded"


def test_concurrent_requests_are_batched(server):
    outs = [None] * 6

    def go(i):
        outs[i] = requests.post(server + "/v1/completions", json={"model": "mock-model", "prompt": f"p{i}", "max_tokens": 12,
                                                                   "temperature": 0}).json()
    ths = [threading.Thread(target=go, args=(i,)) for i in range(6)]
    [t.start() for t in ths]
    [t.join() for t in ths]
    assert all(o["usage"]["completion_tokens"] == 12 for o in outs)


def test_perplexity_and_metrics(server):
    r = requests.post(server + "/v1/perplexity", json={"text": "the quick brown fox jumps over the lazy dog " * 4,
                                                        "chunk_size": 50, "include_token_ppls": True})
    d = r.json()
    assert r.status_code == 200 and d["perplexity"] > 1 and d["tokens"] == len(d["token_ppls"]) and d["chunk_size"] == 50
    assert requests.post(server + "/v1/perplexity", json={"text": ""}).status_code == 400
    assert requests.get(server + "/v1/perplexity/stats").json()["samples"] >= 1
    text = requests.get(server + "/metrics").text
    for name in ("metal_marlin_requests_total", "metal_marlin_latency_ms{quantile=\"0.5\"}", "metal_marlin_tokens_total{type=\"completion\"}",
                 "metal_marlin_queue_depth", "metal_marlin_throughput_tok_sec", "moe_forward_seconds_count",
                 "metal_marlin_perplexity_mean"):
        assert name in text, name
