"""Serving engine: model-format detection, pipeline loading (or a mock model), OpenAI-shaped
completion / chat / streaming entry points, latency statistics.

Parity: reference ``metal_marlin/serving/engine.py``: ``EngineConfig`` ``:472``, ``_detect_model_format``
``:268`` (``mmfp4`` | ``trellis`` | ``marlin``), mock model behind ``METAL_MARLIN_MOCK_MODEL=1`` ``:416-470``,
``chat_completion`` ``:612``, ``_generate`` ``:647`` (request timeout), ``_stream_generate`` ``:788`` (role chunk,
content chunks, stop sequences, final chunk with ``finish_reason``), ``get_latency_stats`` ``:1118``.  Unlike the
reference (whose server never steps its scheduler, ``:1199-1213``), every request here runs on the engine
thread that owns the continuous-batching loop, and trellis checkpoints are served too.
"""
from __future__ import annotations

import asyncio
import json
import os
import time
import uuid
from dataclasses import dataclass, field
from typing import AsyncIterator, Dict, List, Optional

from ..engine.engine import EngineConfig as CoreEngineConfig
from .errors import ContextLengthExceeded, InvalidRequest, ModelNotLoaded, RequestTimeout
from .metrics import MetricsCollector, PerplexityTracker
from .openai_schemas import (ChatChoice, ChatChunkChoice, ChatCompletionChunk, ChatCompletionRequest,
                             ChatCompletionResponse, ChatDelta, ChatMessage, CompletionChoice, CompletionRequest,
                             CompletionResponse, Usage)


@dataclass
class EngineConfig:
    model_path: str = ""
    model_name: Optional[str] = None
    device: Optional[str] = None
    max_model_len: int = 4096
    max_batch_size: int = 32
    request_timeout: float = 60.0
    enable_batching: bool = True
    num_kv_blocks: int = 512
    block_size: int = 16
    use_paged_attention: bool = True
    preset: Optional[str] = None          # serve a random-init architecture preset (no checkpoint)
    speculative: Optional[str] = None     # "ngram" | "mtp" | path of a draft checkpoint
    num_speculative_tokens: int = 4
    kv_cache_dtype: str = "bf16"          # "fp8" | "int8" | "fp4" | "int4": quantized paged cache (one scale per cached row)
    scheduler_policy: str = "priority"    # "priority" | "fcfs" | "shortest_first" | "longest_first"
    preemption_mode: str = "recompute"    # "swap": preempted sequences park their cache rows in pinned host memory
    swap_space_blocks: int = 0
    adaptive_prefill_budget: bool = True   # shrink the prompt-token budget under memory pressure or after an out-of-memory error
    # multi-GPU (job started with torchrun, one process per GPU): tensor / expert / data parallel degrees
    tp: int = 1
    ep: int = 1
    dp: int = 1


def detect_model_format(path: str) -> str:
    """``mmfp4`` | ``trellis`` | ``marlin`` from the files in a checkpoint directory."""
    if not path or not os.path.isdir(path):
        return "marlin"
    if os.path.isdir(os.path.join(path, "layer_0000")) or os.path.exists(os.path.join(path, "quantization_index.json")):
        return "trellis"
    qc = {}
    for fn in ("quantization_config.json", "config.json"):
        p = os.path.join(path, fn)
        if os.path.exists(p):
            with open(p) as f:
                d = json.load(f)
            qc = d if fn.startswith("quantization") else (d.get("quantization_config") or {})
            if qc:
                break
    fmt = str(qc.get("format", qc.get("quant_method", ""))).lower()
    if "trellis" in fmt:
        return "trellis"
    if "mmfp4" in fmt:
        return "mmfp4"
    return "marlin"


class ServingEngine:
    def __init__(self, config: EngineConfig):
        self.config = config
        self.metrics = MetricsCollector()
        self.perplexity_tracker = PerplexityTracker()
        self.mock = os.environ.get("METAL_MARLIN_MOCK_MODEL", "0") == "1"
        self.model_format = "mock" if self.mock else detect_model_format(config.model_path)
        core = CoreEngineConfig(num_kv_blocks=config.num_kv_blocks, block_size=config.block_size,
                                max_model_len=config.max_model_len, max_num_seqs=config.max_batch_size,
                                request_timeout_s=config.request_timeout, kv_cache_dtype=config.kv_cache_dtype,
                                scheduler_policy=config.scheduler_policy, preemption_mode=config.preemption_mode,
                                swap_space_blocks=config.swap_space_blocks,
                                adaptive_prefill_budget=config.adaptive_prefill_budget)
        from ..inference.pipeline import MMFP4Pipeline
        par = dict(tp=config.tp, ep=config.ep, dp=1)        # data-parallel replicas are whole servers behind serving/router.py
        if self.mock:
            self.model_name = config.model_name or os.environ.get("METAL_MARLIN_MOCK_MODEL_NAME", "mock-model")
            self.pipeline = MMFP4Pipeline.from_config("tiny-llama", device="cpu", engine_config=core)
        elif config.preset:
            self.model_name = config.model_name or config.preset
            self.pipeline = MMFP4Pipeline.from_config(config.preset, device=config.device, engine_config=core, **par)
        elif self.model_format == "trellis":
            from ..trellis.lm import TrellisPipeline
            self.model_name = config.model_name or os.path.basename(os.path.normpath(config.model_path))
            self.pipeline = TrellisPipeline.from_pretrained(config.model_path, device=config.device, engine_config=core)
        else:
            self.model_name = config.model_name or os.path.basename(os.path.normpath(config.model_path))
            self.pipeline = MMFP4Pipeline.from_pretrained(config.model_path, device=config.device, engine_config=core, **par)
        if not self.pipeline.is_leader:
            return                      # this rank only executes the leader's batches (see run_server)
        if config.speculative:
            self.pipeline.enable_speculative_decoding(config.speculative, config.num_speculative_tokens)
        self.pipeline.engine.start()

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _stops(stop) -> Optional[List[str]]:
        if stop is None:
            return None
        return [stop] if isinstance(stop, str) else list(stop)

    def _check_len(self, n_prompt: int, n_new: int) -> None:
        if n_prompt + n_new > self.config.max_model_len:
            raise ContextLengthExceeded(f"{n_prompt} prompt tokens + {n_new} requested > max_model_len "
                                        f"{self.config.max_model_len}")

    async def _generate(self, prompt: str, n_new: int, req) -> Dict:
        ids = self.pipeline.encode(prompt)
        self._check_len(len(ids), n_new)
        loop = asyncio.get_running_loop()
        kw = dict(max_new_tokens=n_new, temperature=req.temperature, top_p=req.top_p, top_k=req.top_k,
                  repetition_penalty=req.repetition_penalty, stop=self._stops(req.stop), seed=req.seed or 0, return_ids=True)
        t0 = time.perf_counter()
        try:
            text, out_ids = await asyncio.wait_for(loop.run_in_executor(None, lambda: self.pipeline.generate(prompt, **kw)),
                                                   timeout=self.config.request_timeout)
        except asyncio.TimeoutError:
            raise RequestTimeout(f"request exceeded {self.config.request_timeout}s")
        finish = "length" if len(out_ids) >= n_new and not (out_ids and out_ids[-1] in self.pipeline.eos_ids) else "stop"
        return {"text": text, "prompt_tokens": len(ids), "completion_tokens": len(out_ids), "finish_reason": finish,
                "seconds": time.perf_counter() - t0}

    # ------------------------------------------------------------------ completions
    async def completion(self, req: CompletionRequest) -> CompletionResponse:
        prompts = [req.prompt] if isinstance(req.prompt, str) else list(req.prompt)
        if not prompts or any(not isinstance(p, str) or not p for p in prompts):
            raise InvalidRequest("prompt must be a non-empty string or list of strings")
        t0 = self.metrics.request_started("/v1/completions")
        try:
            results = await asyncio.gather(*[self._generate(p, req.max_tokens, req) for p in prompts for _ in range(req.n)])
        except Exception as e:
            self.metrics.request_finished(t0, error=getattr(e, "code", "internal_error"))
            raise
        choices = [CompletionChoice(index=i, text=(prompts[i // req.n] + r["text"]) if req.echo else r["text"],
                                    finish_reason=r["finish_reason"]) for i, r in enumerate(results)]
        pt, ct = sum(r["prompt_tokens"] for r in results), sum(r["completion_tokens"] for r in results)
        self.metrics.request_finished(t0, pt, ct)
        return CompletionResponse(model=self.model_name, choices=choices,
                                  usage=Usage(prompt_tokens=pt, completion_tokens=ct, total_tokens=pt + ct))

    async def chat_completion(self, req: ChatCompletionRequest) -> ChatCompletionResponse:
        prompt = self.pipeline.format_chat([m.model_dump() for m in req.messages])
        n_new = req.max_tokens or 256
        t0 = self.metrics.request_started("/v1/chat/completions")
        try:
            results = await asyncio.gather(*[self._generate(prompt, n_new, req) for _ in range(req.n)])
        except Exception as e:
            self.metrics.request_finished(t0, error=getattr(e, "code", "internal_error"))
            raise
        choices = [ChatChoice(index=i, message=ChatMessage(role="assistant", content=r["text"]),
                              finish_reason=r["finish_reason"]) for i, r in enumerate(results)]
        pt, ct = results[0]["prompt_tokens"], sum(r["completion_tokens"] for r in results)
        self.metrics.request_finished(t0, pt, ct)
        return ChatCompletionResponse(model=self.model_name, choices=choices,
                                      usage=Usage(prompt_tokens=pt, completion_tokens=ct, total_tokens=pt + ct))

    # ------------------------------------------------------------------ streaming
    async def stream_chat(self, req: ChatCompletionRequest) -> AsyncIterator[ChatCompletionChunk]:
        prompt = self.pipeline.format_chat([m.model_dump() for m in req.messages])
        n_new = req.max_tokens or 256
        n_prompt = len(self.pipeline.encode(prompt))
        self._check_len(n_prompt, n_new)
        cid = "chatcmpl-" + uuid.uuid4().hex[:24]
        t0 = self.metrics.request_started("/v1/chat/completions")
        first = None
        n_out = 0
        yield ChatCompletionChunk(id=cid, model=self.model_name, choices=[ChatChunkChoice(delta=ChatDelta(role="assistant"))])
        finish = "stop"
        async for piece in self.pipeline.astream(prompt, max_new_tokens=n_new, temperature=req.temperature, top_p=req.top_p,
                                                 top_k=req.top_k, repetition_penalty=req.repetition_penalty,
                                                 stop=self._stops(req.stop), seed=req.seed or 0,
                                                 timeout_s=self.config.request_timeout):
            if piece.finished:
                finish = piece.finish_reason or "stop"
                break
            if first is None:
                first = (time.perf_counter() - t0) * 1e3
            n_out += len(piece.token_ids)
            yield ChatCompletionChunk(id=cid, model=self.model_name,
                                      choices=[ChatChunkChoice(delta=ChatDelta(content=piece.text))])
        yield ChatCompletionChunk(id=cid, model=self.model_name,
                                  choices=[ChatChunkChoice(delta=ChatDelta(), finish_reason=finish)])
        self.metrics.request_finished(t0, n_prompt, n_out, ttft_ms=first)

    async def stream_completion(self, req: CompletionRequest) -> AsyncIterator[dict]:
        prompt = req.prompt if isinstance(req.prompt, str) else req.prompt[0]
        n_prompt = len(self.pipeline.encode(prompt))
        self._check_len(n_prompt, req.max_tokens)
        cid = "cmpl-" + uuid.uuid4().hex[:24]
        t0 = self.metrics.request_started("/v1/completions")
        n_out, finish, first = 0, "stop", None
        async for piece in self.pipeline.astream(prompt, max_new_tokens=req.max_tokens, temperature=req.temperature,
                                                 top_p=req.top_p, top_k=req.top_k, stop=self._stops(req.stop),
                                                 seed=req.seed or 0, timeout_s=self.config.request_timeout):
            if piece.finished:
                finish = piece.finish_reason or "stop"
                break
            if first is None:
                first = (time.perf_counter() - t0) * 1e3
            n_out += len(piece.token_ids)
            yield {"id": cid, "object": "text_completion", "created": int(time.time()), "model": self.model_name,
                   "choices": [{"index": 0, "text": piece.text, "finish_reason": None}]}
        yield {"id": cid, "object": "text_completion", "created": int(time.time()), "model": self.model_name,
               "choices": [{"index": 0, "text": "", "finish_reason": finish}]}
        self.metrics.request_finished(t0, n_prompt, n_out, ttft_ms=first)

    # ------------------------------------------------------------------ misc
    def get_latency_stats(self) -> dict:
        return self.metrics.latency_stats()

    def refresh_gauges(self) -> None:
        st = self.pipeline.engine.stats()
        self.metrics.queue_depth = st["waiting"]
        try:
            import torch
            if torch.cuda.is_available():
                self.metrics.gpu_memory_mb = torch.cuda.memory_allocated() / 2 ** 20
        except Exception:
            pass

    def shutdown(self) -> None:
        self.pipeline.close()
