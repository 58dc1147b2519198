"""Pipelined generation: the prompt pass of the next request overlaps the decode steps of the requests that are already
running.  On CUDA the prompt pass is enqueued on its own stream, the decode batch keeps stepping on the main stream and an
event hands the finished prompt over; the KV pool is shared (every request owns a fixed run of blocks), so promoting a
request to the decode batch moves no data.

    sched = PipelineScheduler(lm, max_batch_size=8)
    rid = sched.add_request([1, 2, 3], GenerationConfig(max_new_tokens=16, do_sample=False))
    for request_id, token in sched.generate():
        ...
    outputs = generate_pipelined(lm, [(prompt_a, cfg_a), (prompt_b, None)])      # {index: tensor [1, prompt + new]}

Parity: reference ``metal_marlin/pipeline.py``: ``RequestState`` ``:55``, ``InferenceRequest`` ``:66``, ``PipelineScheduler``
``:87`` (``add_request``, ``generate`` yielding ``(request_id, token)``, ``generate_all``), ``AsyncPipelineScheduler`` ``:290``
(two command queues), ``generate_pipelined`` ``:375``.
"""
from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Iterator, List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..models.mmfp4_causal_lm import prefill
from ..models.transformer import BatchMeta
from ..trellis.generate import GenerationConfig


class RequestState(enum.Enum):
    PENDING_PREFILL = 0
    PREFILLING = 1
    DECODING = 2
    FINISHED = 3


@dataclass
class InferenceRequest:
    request_id: int
    prompt_ids: List[int]
    config: GenerationConfig
    state: RequestState = RequestState.PENDING_PREFILL
    slot: int = -1                                   # which run of cache blocks the request owns
    logits: Optional[torch.Tensor] = None            # [vocab] fp32 of the last position
    generated_ids: List[int] = field(default_factory=list)
    tokens_generated: int = 0
    ready: Optional[object] = None                   # CUDA event recorded after the prompt pass

    @property
    def all_ids(self) -> List[int]:
        return self.prompt_ids + self.generated_ids


class PipelineScheduler:
    """``overlap``: run prompt passes on a second stream (default: on for CUDA models)."""

    def __init__(self, lm, max_batch_size: int = 8, block_size: int = 16, max_model_len: int = 4096, overlap: Optional[bool] = None):
        self.lm, self.model = lm, lm.model
        self.max_batch_size, self.block_size = max_batch_size, block_size
        self.blocks_per_seq = -(-max_model_len // block_size)
        self.max_model_len = self.blocks_per_seq * block_size
        self.device = self.model.device
        self.kv = lm.new_cache(max_batch_size * self.blocks_per_seq, block_size)
        self.tables = torch.arange(max_batch_size * self.blocks_per_seq, dtype=torch.int32).view(max_batch_size, self.blocks_per_seq)
        self.tables_dev = self.tables.to(self.device)
        self.free_slots: List[int] = list(range(max_batch_size))[::-1]
        self.pending_prefill: Deque[InferenceRequest] = deque()
        self.active_decode: List[InferenceRequest] = []
        self.prefilling: Optional[InferenceRequest] = None
        self.finished: List[InferenceRequest] = []
        self._next_id = 0
        self.overlap = (self.device.type == "cuda") if overlap is None else (overlap and self.device.type == "cuda")
        self._side = torch.cuda.Stream(self.device) if self.overlap else None
        self.prefill_steps_overlapped = 0            # decode steps issued while a prompt pass was in flight

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_ids, config: Optional[GenerationConfig] = None) -> int:
        ids = [int(t) for t in (prompt_ids.reshape(-1).tolist() if isinstance(prompt_ids, torch.Tensor) else prompt_ids)]
        cfg = config or GenerationConfig()
        if not ids:
            raise ValueError("empty prompt")
        if len(ids) + cfg.max_new_tokens > self.max_model_len:
            raise ValueError("context_length_exceeded")
        rid = self._next_id
        self._next_id += 1
        self.pending_prefill.append(InferenceRequest(rid, ids, cfg))
        return rid

    # ------------------------------------------------------------------ the two kinds of work
    def _start_prefill(self, r: InferenceRequest) -> None:
        r.state = RequestState.PREFILLING
        r.slot = self.free_slots.pop()
        bt = self.tables[r.slot: r.slot + 1]
        if self._side is not None:
            self._side.wait_stream(torch.cuda.current_stream(self.device))       # the slot's previous owner has finished reading it
            with torch.cuda.stream(self._side):
                r.logits = prefill(self.model, self.kv, [r.prompt_ids], bt)[0]
                r.ready = torch.cuda.Event()
                r.ready.record(self._side)
        else:
            r.logits = prefill(self.model, self.kv, [r.prompt_ids], bt)[0]

    def _prefill_done(self, r: InferenceRequest) -> bool:
        return r.ready is None or r.ready.query()

    def _promote(self, r: InferenceRequest) -> None:
        if r.ready is not None:
            torch.cuda.current_stream(self.device).wait_event(r.ready)
            r.ready = None
        r.state = RequestState.DECODING
        self.active_decode.append(r)

    def _sample(self, rs: Sequence[InferenceRequest], logits: torch.Tensor) -> List[int]:
        """One token per request from ``logits [n, vocab]`` under each request's own configuration."""
        greedy = [(not r.config.do_sample) or r.config.temperature == 0 for r in rs]
        plain = all(g and r.config.repetition_penalty == 1.0 for g, r in zip(greedy, rs))
        if plain:
            return [int(t) for t in self.model.greedy(logits).tolist()]
        dev = logits.device
        full = self.model.full_logits(logits)
        H = max(1, max(len(r.all_ids) for r in rs))
        hist = torch.full((len(rs), H), -1, dtype=torch.int64)
        for i, r in enumerate(rs):
            a = r.all_ids
            hist[i, : len(a)] = torch.tensor(a, dtype=torch.int64)
        f = lambda vals, dt: torch.tensor(vals, dtype=dt, device=dev)
        ids = ops.sample(full, temperature=f([0.0 if g else r.config.temperature for g, r in zip(greedy, rs)], torch.float32),
                         top_k=f([r.config.top_k for r in rs], torch.int32), top_p=f([r.config.top_p for r in rs], torch.float32),
                         min_p=f([0.0] * len(rs), torch.float32), history=hist.to(dev),
                         rep_penalty=f([r.config.repetition_penalty for r in rs], torch.float32),
                         seed=rs[0].config.seed, offset=rs[0].tokens_generated,
                         seed_dev=f([r.config.seed + r.request_id for r in rs], torch.int64) if dev.type == "cuda" else None)
        return [int(t) for t in ids.tolist()]

    def _decode_step(self) -> List[Tuple[int, int]]:
        """Sample one token for every active request from its current logits, then run ONE batched forward for the survivors."""
        rs = self.active_decode
        toks = self._sample(rs, torch.stack([r.logits for r in rs]))
        out, cont = [], []
        for r, t in zip(rs, toks):
            eos = r.config.eos_token_id
            eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
            r.tokens_generated += 1
            r.generated_ids.append(t)
            out.append((r.request_id, t))
            if t in eos or r.tokens_generated >= r.config.max_new_tokens:
                r.state = RequestState.FINISHED
                r.logits = None
                self.free_slots.append(r.slot)
                self.finished.append(r)
            else:
                cont.append(r)
        self.active_decode = cont
        if cont:
            dev, bs = self.device, self.block_size
            pos = [len(r.all_ids) - 1 for r in cont]                 # position of the token just sampled
            slots = [int(self.tables[r.slot, p // bs]) * bs + p % bs for r, p in zip(cont, pos)]
            meta = BatchMeta(positions=torch.tensor(pos, dtype=torch.int32, device=dev), slots=torch.tensor(slots, dtype=torch.int64, device=dev),
                             block_tables=self.tables_dev[[r.slot for r in cont]].contiguous(),
                             ctx_lens=torch.tensor([p + 1 for p in pos], dtype=torch.int32, device=dev), decode=True,
                             max_ctx=self.max_model_len)
            logits = self.model.forward(torch.tensor([r.generated_ids[-1] for r in cont], dtype=torch.int64, device=dev), self.kv, meta)
            for i, r in enumerate(cont):
                r.logits = logits[i]
        return out

    # ------------------------------------------------------------------ the loop
    def generate(self) -> Iterator[Tuple[int, int]]:
        while self.pending_prefill or self.active_decode or self.prefilling is not None:
            if self.prefilling is None and self.pending_prefill and self.free_slots:
                self.prefilling = self.pending_prefill.popleft()
                self._start_prefill(self.prefilling)
            if self.prefilling is not None and (self._prefill_done(self.prefilling) or not self.active_decode):
                self._promote(self.prefilling)
                self.prefilling = None
                if self.pending_prefill and self.free_slots and len(self.active_decode) < self.max_batch_size:
                    continue                                         # start the next prompt pass before stepping
            if self.active_decode:
                if self.prefilling is not None:
                    self.prefill_steps_overlapped += 1
                for pair in self._decode_step():
                    yield pair

    def generate_all(self) -> Dict[int, torch.Tensor]:
        for _ in self.generate():
            pass
        return {r.request_id: torch.tensor([r.all_ids], dtype=torch.long, device=self.device) for r in self.finished}


class AsyncPipelineScheduler(PipelineScheduler):
    """Always asks for the two-stream overlap (a CPU model falls back to alternating prompt passes and decode steps)."""

    def __init__(self, lm, max_batch_size: int = 8, block_size: int = 16, max_model_len: int = 4096):
        super().__init__(lm, max_batch_size, block_size, max_model_len, overlap=True)


def generate_pipelined(lm, requests: Sequence[Tuple[Sequence[int], Optional[GenerationConfig]]], max_batch_size: int = 8,
                       max_model_len: Optional[int] = None) -> Dict[int, torch.Tensor]:
    """Run all requests through a ``PipelineScheduler``; returns ``{index in requests: ids [1, prompt + new]}``."""
    need = max(len(p if not isinstance(p, torch.Tensor) else p.reshape(-1)) + (c or GenerationConfig()).max_new_tokens for p, c in requests)
    sched = PipelineScheduler(lm, max_batch_size=max_batch_size, max_model_len=max_model_len or need)
    index = {sched.add_request(p, c): i for i, (p, c) in enumerate(requests)}
    return {index[rid]: t for rid, t in sched.generate_all().items()}
