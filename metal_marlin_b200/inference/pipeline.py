"""``MMFP4Pipeline``: text in, text out.

Parity: reference ``metal_marlin/inference/mmfp4_pipeline.py:1238-3158`` — ``from_pretrained`` ``:1810``,
``__call__`` ``:1872`` / ``generate`` ``:1890`` (exact-match result cache ``:1904``, streaming ``:1984``),
``chat`` ``:2080``, ``chat_stream`` ``:2695``, ``enable_speculative_decoding`` ``:1303``, prefix-matched
persistent KV (``PersistentKVCache`` ``:31``, ``_match_cache_prefix`` ``:1624``), dynamic batching ``:2735``;
and ``MarlinPipeline`` (``metal_marlin/inference/pipeline.py:835``) for dense ``marlin_fp4`` checkpoints —
the same class serves both formats here because the loader normalises them.

All generation goes through :class:`LLMEngine` (paged cache, prefix reuse across calls, continuous
batching of concurrent calls); streaming hands tokens over a queue from the engine thread.
"""
from __future__ import annotations

import asyncio
import queue
import threading
import time
from collections import OrderedDict
from dataclasses import dataclass
from typing import AsyncIterator, Dict, Iterator, List, Optional, Sequence, Union

import torch

from ..engine.engine import EngineConfig, LLMEngine
from ..engine.request import GenerationRequest, RequestPriority, RunningRequest
from ..engine.session import SamplingParams
from ..models.config import ModelConfig
from ..models.mmfp4_causal_lm import MMFP4ForCausalLM
from .tokenizer import load_tokenizer


@dataclass
class StreamingOutput:
    """One streamed piece.  ``finished`` is set on the last item, with the finish reason."""
    text: str
    token_ids: List[int]
    finished: bool = False
    finish_reason: Optional[str] = None


class _IncrementalDecoder:
    """Turns a growing id list into text pieces without splitting multi-byte characters."""

    def __init__(self, tok):
        self.tok, self.ids, self.emitted = tok, [], ""

    def push(self, tid: int) -> str:
        self.ids.append(tid)
        text = self.tok.decode(self.ids, skip_special_tokens=True)
        if text.endswith("�"):
            return ""
        piece = text[len(self.emitted):]
        self.emitted = text
        return piece


class MMFP4Pipeline:
    def __init__(self, model: MMFP4ForCausalLM, tokenizer, engine_config: Optional[EngineConfig] = None,
                 result_cache_size: int = 64, parallel=None):
        """``parallel``: an ``engine.distributed.ParallelConfig`` (or a dict ``{"tp": .., "ep": .., "dp": ..}``) in a job
        started with ``torchrun``: the model is sharded over the ranks, rank 0 drives generation through the same calls
        as on one GPU and every other rank calls :meth:`serve_forever`."""
        self.model, self.tokenizer = model, tokenizer
        self.config: ModelConfig = model.config
        self.device = model.device
        ec = engine_config or EngineConfig(max_model_len=min(self.config.max_position_embeddings, 8192))
        self.parallel = None
        if parallel is not None and not (isinstance(parallel, dict) and not any(v and v > 1 for v in parallel.values())):
            from ..engine.distributed import ParallelConfig, build_engine, init_process_group
            rank, world, dev, ctrl = init_process_group(torch.device(self.device))
            pc = parallel if isinstance(parallel, ParallelConfig) else ParallelConfig.parse(world=world, **parallel)
            self.parallel = pc
            self.rank, self.world = rank, world
            if pc.mode in ("single", "dp"):
                self.engine = LLMEngine(model.model, ec)
            else:
                self.engine = build_engine(model.model, ec, pc, rank, world, dev, ctrl)
                model.model = self.engine.model          # the rank's shard; the whole model is released
        else:
            self.engine = LLMEngine(model.model, ec)
        self._results: "OrderedDict[tuple, str]" = OrderedDict()
        self._result_cache_size = result_cache_size
        self.speculative = None
        self._spec_args = None
        self.stats = {"requests": 0, "prompt_tokens": 0, "completion_tokens": 0}

    # ------------------------------------------------------------------ construction
    @staticmethod
    def _parallel_args(tp, ep, dp, device):
        """(parallel dict or None, device): in a multi-rank job every rank loads onto its own GPU."""
        import os
        if max(tp, ep, dp) <= 1:
            return None, device
        if device is None and torch.cuda.is_available():
            device = f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}"
        return {"tp": tp, "ep": ep, "dp": dp}, device

    @classmethod
    def from_pretrained(cls, path: str, device: Optional[str] = None, engine_config: Optional[EngineConfig] = None,
                        tp: int = 1, ep: int = 1, dp: int = 1, **_ignored) -> "MMFP4Pipeline":
        par, device = cls._parallel_args(tp, ep, dp, device)
        lm = MMFP4ForCausalLM.from_pretrained(path, device)
        return cls(lm, load_tokenizer(path, lm.config.vocab_size), engine_config, parallel=par)

    @classmethod
    def from_config(cls, cfg, device: Optional[str] = None, seed: int = 0,
                    engine_config: Optional[EngineConfig] = None, tp: int = 1, ep: int = 1, dp: int = 1) -> "MMFP4Pipeline":
        par, device = cls._parallel_args(tp, ep, dp, device)
        lm = MMFP4ForCausalLM.from_config(cfg, device, seed)
        return cls(lm, load_tokenizer(None, lm.config.vocab_size), engine_config, parallel=par)

    @property
    def is_leader(self) -> bool:
        """False on the ranks of a multi-GPU job that only execute what rank 0 schedules."""
        return getattr(self.engine, "is_leader", True)

    def serve_forever(self) -> None:
        """Ranks other than 0 of a tensor- / expert-parallel job: run the leader's batches until it closes the pipeline."""
        if hasattr(self.engine, "serve_forever"):
            self.engine.serve_forever()

    # ------------------------------------------------------------------ helpers
    @property
    def eos_ids(self) -> List[int]:
        e = getattr(self.tokenizer, "eos_token_id", None)
        if e is None:
            return []
        return [e] if isinstance(e, int) else list(e)

    def encode(self, text: str) -> List[int]:
        ids = self.tokenizer.encode(text) if hasattr(self.tokenizer, "encode") else self.tokenizer(text)["input_ids"]
        v = self.config.vocab_size
        return [i if i < v else i % v for i in ids]

    def _sampling(self, temperature, top_p, top_k, repetition_penalty=1.0, min_p=0.0, seed=0) -> SamplingParams:
        return SamplingParams(temperature=float(temperature or 0.0), top_k=int(top_k or 0), top_p=float(top_p or 1.0),
                              min_p=float(min_p or 0.0), repetition_penalty=float(repetition_penalty or 1.0), seed=seed)

    def _ensure_thread(self):
        self.engine.start()

    @staticmethod
    def _apply_stop(text: str, stop: Optional[Sequence[str]]):
        if not stop:
            return text, False
        cut = min((text.find(s) for s in stop if s and s in text), default=-1)
        return (text[:cut], True) if cut >= 0 else (text, False)

    # ------------------------------------------------------------------ generation
    def __call__(self, prompt: Union[str, Sequence[str]], **kw):
        return self.generate(prompt, **kw)

    def generate(self, prompt: Union[str, Sequence[str]], max_new_tokens: Optional[int] = None, max_tokens: Optional[int] = None,
                 temperature: float = 0.0, top_p: float = 1.0, top_k: int = 0, repetition_penalty: float = 1.0,
                 min_p: float = 0.0, stop: Optional[Sequence[str]] = None, stream: bool = False, seed: int = 0,
                 priority: RequestPriority = RequestPriority.NORMAL, return_ids: bool = False):
        n_new = max_new_tokens or max_tokens or 64
        if isinstance(prompt, (list, tuple)):
            if stream:
                raise ValueError("stream=True takes a single prompt")
            return self.generate_batch(list(prompt), n_new, temperature, top_p, top_k, repetition_penalty, min_p, stop, seed)
        if stream:
            return self.stream(prompt, n_new, temperature, top_p, top_k, repetition_penalty, min_p, stop, seed, priority)
        key = (prompt, n_new, temperature, top_p, top_k, repetition_penalty, min_p, tuple(stop or ()), seed)
        if temperature <= 0 and key in self._results and not return_ids:
            self._results.move_to_end(key)
            return self._results[key]
        rr = self._submit(self.encode(prompt), n_new, self._sampling(temperature, top_p, top_k, repetition_penalty, min_p, seed),
                          priority)
        self._wait([rr])
        ids = [t for t in rr.output_ids if t not in self.eos_ids]
        text, _ = self._apply_stop(self.tokenizer.decode(ids, skip_special_tokens=True), stop)
        if temperature <= 0:
            self._results[key] = text
            while len(self._results) > self._result_cache_size:
                self._results.popitem(last=False)
        return (text, rr.output_ids) if return_ids else text

    def generate_batch(self, prompts: List[str], max_new_tokens=64, temperature=0.0, top_p=1.0, top_k=0,
                       repetition_penalty=1.0, min_p=0.0, stop=None, seed=0) -> List[str]:
        sp = self._sampling(temperature, top_p, top_k, repetition_penalty, min_p, seed)
        rrs = [self._submit(self.encode(p), max_new_tokens, sp) for p in prompts]
        self._wait(rrs)
        outs = []
        for rr in rrs:
            ids = [t for t in rr.output_ids if t not in self.eos_ids]
            outs.append(self._apply_stop(self.tokenizer.decode(ids, skip_special_tokens=True), stop)[0])
        return outs

    def _submit(self, ids: List[int], n_new: int, sp: SamplingParams, priority=RequestPriority.NORMAL, on_token=None
                ) -> RunningRequest:
        max_len = self.engine.cfg.max_model_len
        if len(ids) + n_new > max_len:
            raise ValueError(f"context_length_exceeded: {len(ids)} prompt + {n_new} new > {max_len}")
        self.stats["requests"] += 1
        self.stats["prompt_tokens"] += len(ids)
        return self.engine.add_request(GenerationRequest(ids, n_new, sp, eos_ids=self.eos_ids, priority=priority,
                                                         on_token=on_token))

    def _wait(self, rrs: List[RunningRequest]) -> None:
        if self.engine._thread is None:
            self.engine.run_until_done()
        for rr in rrs:
            rr.done.wait()
            self.stats["completion_tokens"] += len(rr.output_ids)
            if rr.error:
                raise RuntimeError(rr.error)

    # ------------------------------------------------------------------ streaming
    def stream(self, prompt: str, max_new_tokens=64, temperature=0.0, top_p=1.0, top_k=0, repetition_penalty=1.0,
               min_p=0.0, stop=None, seed=0, priority=RequestPriority.NORMAL, timeout_s: float = 60.0
               ) -> Iterator[StreamingOutput]:
        """Generator of :class:`StreamingOutput`; tokens are produced by the engine thread."""
        self._ensure_thread()
        q: "queue.Queue" = queue.Queue()
        rr = self._submit(self.encode(prompt), max_new_tokens,
                          self._sampling(temperature, top_p, top_k, repetition_penalty, min_p, seed), priority,
                          on_token=lambda rid, t: q.put(t))
        dec = _IncrementalDecoder(self.tokenizer)
        emitted = ""
        deadline = time.monotonic() + timeout_s
        n_seen = 0
        while True:
            try:
                tok = q.get(timeout=0.05)
            except queue.Empty:
                if rr.done.is_set() and q.empty():
                    break
                if time.monotonic() > deadline:
                    self.engine.abort(rr.id)
                    yield StreamingOutput("", [], True, "timeout")
                    return
                continue
            n_seen += 1
            if tok in self.eos_ids:
                continue
            piece = dec.push(tok)
            if not piece:
                continue
            full, hit = self._apply_stop(emitted + piece, stop)
            piece = full[len(emitted):]
            emitted = full
            if piece:
                yield StreamingOutput(piece, [tok])
            if hit:
                self.engine.abort(rr.id)
                yield StreamingOutput("", [], True, "stop")
                return
        self.stats["completion_tokens"] += len(rr.output_ids)
        yield StreamingOutput("", [], True, rr.finish_reason or "stop")

    async def astream(self, prompt: str, **kw) -> AsyncIterator[StreamingOutput]:
        """Async wrapper: the blocking generator runs in a worker thread, pieces cross an asyncio.Queue."""
        loop = asyncio.get_running_loop()
        aq: asyncio.Queue = asyncio.Queue()
        DONE = object()

        def pump():
            try:
                for item in self.stream(prompt, **kw):
                    loop.call_soon_threadsafe(aq.put_nowait, item)
            except Exception as e:   # surface engine errors to the consumer
                loop.call_soon_threadsafe(aq.put_nowait, e)
            loop.call_soon_threadsafe(aq.put_nowait, DONE)

        threading.Thread(target=pump, daemon=True).start()
        while True:
            item = await aq.get()
            if item is DONE:
                return
            if isinstance(item, Exception):
                raise item
            yield item

    # ------------------------------------------------------------------ chat
    def format_chat(self, messages: Sequence[Dict[str, str]]) -> str:
        if hasattr(self.tokenizer, "apply_chat_template"):
            try:
                return self.tokenizer.apply_chat_template(list(messages), add_generation_prompt=True, tokenize=False)
            except Exception:
                pass
        return "".join(f"<|{m['role']}|>\n{m['content']}\n" for m in messages) + "<|assistant|>\n"

    def chat(self, messages: Sequence[Dict[str, str]], **kw) -> str:
        return self.generate(self.format_chat(messages), **kw)

    def chat_stream(self, messages: Sequence[Dict[str, str]], **kw) -> Iterator[StreamingOutput]:
        return self.stream(self.format_chat(messages), **kw)

    # ------------------------------------------------------------------ speculative decoding
    def enable_speculative_decoding(self, draft="ngram", num_speculative_tokens: int = 4, **kw) -> None:
        """Attach a draft source.  ``draft``: ``"ngram"``, ``"mtp"``, ``"eagle"``, the path of a small checkpoint, a small
        :class:`MMFP4ForCausalLM`, or any object implementing ``spec.draft.DraftModel``.

        N-gram and small-model drafts run inside the continuous-batching engine: every generate / stream / server call
        then drafts and verifies per step, batched over all running requests.  Drafts that need the target's hidden state
        (MTP, EAGLE trees) serve :meth:`speculative_generate` (one request at a time)."""
        from ..spec.draft import DraftModel
        self._spec_args = (draft, num_speculative_tokens, kw)
        self.speculative = None
        core = getattr(self.engine, "engine", self.engine)          # a multi-GPU engine wraps the rank's LLMEngine
        if isinstance(draft, str) and draft not in ("ngram", "mtp", "eagle"):
            draft = MMFP4ForCausalLM.from_pretrained(draft, str(self.device))
            self._spec_args = (draft, num_speculative_tokens, kw)
        if draft == "ngram" or isinstance(draft, MMFP4ForCausalLM):
            core.enable_speculative(draft, num_speculative_tokens, **kw)
            self._results.clear()
        elif isinstance(draft, DraftModel) or draft in ("mtp", "eagle"):
            self._ensure_spec_engine()

    def _ensure_spec_engine(self):
        if self.speculative is None:
            if getattr(self, "_spec_args", None) is None:
                raise RuntimeError("call enable_speculative_decoding() first")
            from ..spec.engine import SpeculativeEngine, make_draft
            draft, k, kw = self._spec_args
            self.speculative = SpeculativeEngine(self.model, make_draft(draft, self.model, **kw), num_speculative_tokens=k)
        return self.speculative

    def speculative_generate(self, prompt: str, max_new_tokens: int = 64, temperature: float = 0.0, seed: int = 0):
        spec = self._ensure_spec_engine()
        ids, stats = spec.generate(self.encode(prompt), max_new_tokens, temperature=temperature, seed=seed, eos_ids=self.eos_ids)
        return self.tokenizer.decode([t for t in ids if t not in self.eos_ids], skip_special_tokens=True), stats

    def speculative_stats(self) -> dict:
        """Acceptance statistics of the in-engine speculative decoding."""
        st = getattr(self.engine, "engine", self.engine).stats()
        return {k: st[k] for k in ("spec_proposed", "spec_accepted", "spec_acceptance_rate") if k in st}

    # ------------------------------------------------------------------ perplexity
    @torch.no_grad()
    def token_nll(self, text_or_ids: Union[str, Sequence[int]]) -> torch.Tensor:
        ids = self.encode(text_or_ids) if isinstance(text_or_ids, str) else list(text_or_ids)
        if len(ids) < 2:
            return torch.zeros(0)
        logits = self.model.forward_logits(ids)
        lp = torch.log_softmax(logits[:-1].float(), -1)
        tgt = torch.tensor(ids[1:], device=lp.device)
        return -lp.gather(1, tgt.unsqueeze(1)).squeeze(1).cpu()

    def close(self) -> None:
        self.engine.stop()


# the dense marlin_fp4 pipeline of the reference is the same object here
class MarlinPipeline(MMFP4Pipeline):
    """The generic pipeline surface over the same engine: ``from_pretrained(path, quant_type=...)`` for dense ``marlin_fp4`` /
    MMFP4 checkpoints, ``__call__``, ``stream_generate`` / ``generate_stream`` (text chunks), ``generate_batch``, ``chat`` and
    ``info()``.  Parity: reference ``metal_marlin/inference/pipeline.py:835`` (``MarlinPipeline``), ``:901`` (``__call__``),
    ``:918`` (``stream_generate``), ``:932`` (``info``), ``metal_marlin/inference/pipeline_v2.py`` (``TransformersMarlinPipeline``)."""

    @classmethod
    def from_pretrained(cls, path: str, quant_type: str = "fp4", device: Optional[str] = None, **kw):
        if quant_type not in ("fp4", "mmfp4", "marlin_fp4"):
            import warnings
            warnings.warn(f"quant_type={quant_type!r}: checkpoints are read in the format they were written in", UserWarning, stacklevel=2)
        return super().from_pretrained(path, device=device, **kw)

    def stream_generate(self, prompt: str, max_tokens: int = 64, **kw) -> Iterator[str]:
        for chunk in self.stream(prompt, max_new_tokens=max_tokens, **kw):
            if chunk.text:
                yield chunk.text

    generate_stream = stream_generate

    def info(self) -> Dict[str, object]:
        cfg = self.config
        m = self.model.model
        return {"model_type": cfg.model_type, "num_layers": cfg.num_hidden_layers, "hidden_size": cfg.hidden_size,
                "vocab_size": cfg.vocab_size, "num_attention_heads": cfg.num_attention_heads, "num_experts": getattr(cfg, "num_experts", 0) or 0,
                "attention": "mla" if cfg.is_mla else "gqa", "quant_format": getattr(cfg, "quant_format", "mmfp4"), "group_size": cfg.group_size,
                "weight_bytes": int(m.weight_bytes()), "device": str(self.device), "max_model_len": self.engine.cfg.max_model_len}
