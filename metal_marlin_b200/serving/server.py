"""OpenAI-compatible HTTP server (FastAPI).

Routes (same paths, payloads, SSE framing and error envelope as the reference,
``metal_marlin/serving/server.py:90-247``): ``GET /v1/models``, ``GET /v1/models/{id}``,
``POST /v1/chat/completions``, ``POST /v1/completions`` (``stream=true`` -> ``data: {json}\\n\\n`` ...
``data: [DONE]\\n\\n``), ``GET /health``, ``POST /v1/perplexity``, ``GET /v1/perplexity/stats``,
``GET /metrics`` (Prometheus text).  ``run_server`` (``:250``) optionally exposes ``/metrics`` on a second port.
"""
from __future__ import annotations

import json
import threading
from typing import Optional

from fastapi import FastAPI, Request
from fastapi.exceptions import RequestValidationError
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from .engine import EngineConfig, ServingEngine
from .errors import InvalidRequest, ModelNotFound, ModelNotLoaded, ServingError
from .metrics import moe_metrics
from .openai_schemas import (ChatCompletionRequest, CompletionRequest, ModelInfo, ModelList, PerplexityRequest,
                             PerplexityResponse)
from .perplexity import compute_perplexity

app = FastAPI(title="metal-marlin (B200)", version="0.1.0")
_engine: Optional[ServingEngine] = None


def configure(config: EngineConfig) -> ServingEngine:
    global _engine
    if _engine is not None:
        _engine.shutdown()
    _engine = ServingEngine(config)
    return _engine


def get_engine() -> ServingEngine:
    if _engine is None:
        raise ModelNotLoaded("no model is loaded")
    return _engine


@app.exception_handler(ServingError)
async def _serving_error(_: Request, exc: ServingError):
    return JSONResponse(status_code=exc.status_code, content=exc.to_dict())


@app.exception_handler(RequestValidationError)
async def _validation_error(_: Request, exc: RequestValidationError):
    return JSONResponse(status_code=422, content={"error": {"message": str(exc.errors()), "type": "invalid_request_error",
                                                            "code": "validation_error"}})


def _check_model(name: Optional[str], eng: ServingEngine) -> None:
    if name is not None and name != eng.model_name:
        raise ModelNotFound(f"model {name!r} not found; serving {eng.model_name!r}")


@app.get("/health")
async def health():
    return {"status": "ok", "model_loaded": _engine is not None,
            "engine_error": None if _engine is None else _engine.pipeline.engine.last_error}


@app.get("/v1/models")
async def list_models():
    eng = get_engine()
    return ModelList(data=[ModelInfo(id=eng.model_name)])


@app.get("/v1/models/{model_id}")
async def get_model(model_id: str):
    eng = get_engine()
    _check_model(model_id, eng)
    return ModelInfo(id=eng.model_name)


def _sse(gen):
    async def body():
        async for item in gen:
            payload = item.model_dump_json(exclude_none=False) if hasattr(item, "model_dump_json") else json.dumps(item)
            yield f"data: {payload}\n\n"
        yield "data: [DONE]\n\n"
    return StreamingResponse(body(), media_type="text/event-stream")


@app.post("/v1/chat/completions")
async def chat_completions(req: ChatCompletionRequest):
    eng = get_engine()
    _check_model(req.model, eng)
    if req.stream:
        return _sse(eng.stream_chat(req))
    return await eng.chat_completion(req)


@app.post("/v1/completions")
async def completions(req: CompletionRequest):
    eng = get_engine()
    _check_model(req.model, eng)
    if req.stream:
        return _sse(eng.stream_completion(req))
    return await eng.completion(req)


@app.post("/v1/perplexity")
async def perplexity(req: PerplexityRequest):
    eng = get_engine()
    _check_model(req.model, eng)
    try:
        res = compute_perplexity(eng.pipeline, req.text, req.chunk_size, req.include_token_ppls)
    except ValueError as e:
        raise InvalidRequest(str(e))
    eng.perplexity_tracker.record(res["perplexity"], res["tokens"])
    return PerplexityResponse(**res)


@app.get("/v1/perplexity/stats")
async def perplexity_stats():
    return get_engine().perplexity_tracker.stats()


def metrics_text() -> str:
    eng = get_engine()
    eng.refresh_gauges()
    return eng.metrics.to_prometheus() + moe_metrics.to_prometheus() + eng.perplexity_tracker.to_prometheus()


@app.get("/metrics")
async def metrics():
    return PlainTextResponse(metrics_text(), media_type="text/plain; version=0.0.4")


def run_server(config: EngineConfig, host: str = "127.0.0.1", port: int = 8000, metrics_port: Optional[int] = None,
               log_level: str = "info") -> None:
    import os

    import uvicorn
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if config.dp > 1 and config.tp == 1 and config.ep == 1:
        # data parallel: every rank is a whole replica with its own server on port + 1 + rank; rank 0 also runs the router
        if world != config.dp:
            raise ValueError(f"--dp {config.dp} needs {config.dp} processes (torchrun), the job has {world}")
        if config.device is None:
            config.device = f"cuda:{os.environ.get('LOCAL_RANK', '0')}"
        if rank == 0:
            from .router import run_router
            backends = [f"http://{host}:{port + 1 + r}" for r in range(world)]
            threading.Thread(target=lambda: run_router(backends, host=host, port=port, log_level="warning"), daemon=True).start()
        port = port + 1 + rank
    eng = configure(config)
    if not eng.pipeline.is_leader:
        try:
            eng.pipeline.serve_forever()         # tensor / expert parallel: execute what rank 0 schedules
        finally:
            return
    if metrics_port:
        mapp = FastAPI()
        mapp.get("/metrics")(metrics)
        threading.Thread(target=lambda: uvicorn.run(mapp, host=host, port=metrics_port, log_level="warning"),
                         daemon=True).start()
    try:
        uvicorn.run(app, host=host, port=port, log_level=log_level)
    finally:
        if _engine is not None:
            _engine.shutdown()
