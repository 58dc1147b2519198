"""Continuous-batching scheduler: per-iteration token budgets, decode-first planning, chunked
prefill, priorities with starvation promotion, preemption by recompute or by swapping the victim's cache blocks to host
memory (``preemption_mode="swap"``: the scheduler plans the block moves, the engine copies).  The first-come-first-served scheduler with
prefill strategies and insertion policies builds on it in ``engine/fcfs.py``.

Parity: reference ``metal_marlin/serving/continuous_batch.py``: ``SchedulerConfig`` (max_num_seqs 64,
max_num_batched_tokens 2048, max_prefill_tokens 1024, chunk 512, starvation 30 s), ``PreemptionPolicy``,
``IterationPlanner.plan_iteration`` ``:374`` (phase 1: one decode token per running sequence, phase 2:
prefill chunks inside the remaining budget), ``BatchScheduler.schedule`` ``:550`` / ``step`` ``:614`` /
``_preempt`` ``:663`` / ``_check_starvation`` ``:698``; ``metal_marlin/serving/scheduler.py:329``
(``FCFSScheduler``, queue-full error, insertion policies).
"""
from __future__ import annotations

import enum
import heapq
import itertools
import time
from dataclasses import dataclass
from typing import Dict, List, Optional

from ..kv.paged import OutOfBlocks, PagedKVCache
from .request import (GenerationRequest, PrefillChunk, RequestPriority, RequestStatus, RunningRequest,
                      SchedulerOutput)


class PreemptionPolicy(enum.Enum):
    MOST_TOKENS = "most_tokens"
    LEAST_TOKENS = "least_tokens"
    OLDEST = "oldest"
    LOWEST_PRIORITY = "lowest_priority"


class QueueFullError(RuntimeError):
    pass


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 2048
    max_prefill_tokens: int = 1024
    block_size: int = 16
    enable_chunked_prefill: bool = True
    max_chunk: int = 512
    starvation_s: float = 30.0
    preemption_policy: PreemptionPolicy = PreemptionPolicy.LOWEST_PRIORITY
    max_waiting: int = 4096
    max_model_len: int = 1 << 20
    fcfs: bool = False                     # ignore priorities: strict arrival order
    preemption_mode: str = "recompute"     # "swap": a fully prefilled victim keeps its cache rows in host blocks
    swap_space_blocks: int = 0             # host blocks available to swapped sequences
    proactive_evict_above: float = 0.9     # cached prefix blocks are released while more than this share of the pool is in use


class BatchScheduler:
    def __init__(self, config: SchedulerConfig, cache: PagedKVCache):
        self.cfg, self.cache = config, cache
        self._heap: List = []
        self._seq = itertools.count()
        self.running: List[RunningRequest] = []
        self.requests: Dict[str, RunningRequest] = {}
        self.num_preemptions = 0
        self.num_finished = 0
        self.swapped_out: List[RunningRequest] = []          # sequences whose cache rows sit in host blocks, oldest first
        self._host_free: List[int] = list(range(config.swap_space_blocks if config.preemption_mode == "swap" else 0))
        self.num_swaps = 0

    # ------------------------------------------------------------------ queue
    def add_request(self, req: GenerationRequest) -> RunningRequest:
        if self.num_waiting >= self.cfg.max_waiting:
            raise QueueFullError(f"waiting queue is full ({self.cfg.max_waiting})")
        if len(req.prompt_ids) + req.max_new_tokens > self.cfg.max_model_len:
            raise ValueError("context_length_exceeded")
        rr = RunningRequest(req)
        self.requests[rr.id] = rr
        self._push(rr)
        return rr

    def _push(self, rr: RunningRequest) -> None:
        pr = 0 if self.cfg.fcfs else -rr.effective_priority
        heapq.heappush(self._heap, (pr, rr.arrival, next(self._seq), rr))

    def _peek_waiting(self) -> Optional[RunningRequest]:
        """The request admission looks at next (the head of the queue blocks the ones behind it)."""
        return self._heap[0][3] if self._heap else None

    def _pop_waiting(self, rr: RunningRequest) -> None:
        assert self._heap[0][3] is rr
        heapq.heappop(self._heap)

    def _drop_waiting(self, rr: RunningRequest) -> None:
        self._heap = [e for e in self._heap if e[3] is not rr]
        heapq.heapify(self._heap)

    @property
    def num_waiting(self) -> int:
        return len(self._heap)

    def has_work(self) -> bool:
        return bool(self._heap or self.running or self.swapped_out)

    def abort(self, request_id: str) -> bool:
        rr = self.requests.get(request_id)
        if rr is None or rr.status in (RequestStatus.FINISHED, RequestStatus.ABORTED, RequestStatus.FAILED):
            return False
        if rr in self.running:
            self.running.remove(rr)
            self.cache.release(rr.id)
        elif rr in self.swapped_out:
            self.swapped_out.remove(rr)
            self._host_free.extend(rr.swap_host_blocks)
            rr.swap_host_blocks = None
        else:
            self._drop_waiting(rr)
            if self.cache.table.has(rr.id):
                self.cache.release(rr.id)
        rr.finish_reason = "abort"
        rr.transition(RequestStatus.ABORTED)
        return True

    # ------------------------------------------------------------------ policy helpers
    def _check_starvation(self) -> None:
        if self.cfg.fcfs:
            return
        now = time.monotonic()
        changed = False
        for i, (pr, arr, seq, rr) in enumerate(self._heap):
            if now - arr > self.cfg.starvation_s and rr.effective_priority < int(RequestPriority.REALTIME):
                rr.effective_priority += 1
                self._heap[i] = (-rr.effective_priority, now, seq, rr)     # restart its clock after a promotion
                changed = True
        if changed:
            heapq.heapify(self._heap)

    def _pick_victim(self, exclude=()) -> Optional[RunningRequest]:
        cands = [r for r in self.running if r not in exclude]
        if not cands:
            return None
        pol = self.cfg.preemption_policy
        if pol is PreemptionPolicy.MOST_TOKENS:
            return max(cands, key=lambda r: len(r.all_ids))
        if pol is PreemptionPolicy.LEAST_TOKENS:
            return min(cands, key=lambda r: len(r.all_ids))
        if pol is PreemptionPolicy.OLDEST:
            return min(cands, key=lambda r: r.arrival)
        return min(cands, key=lambda r: (r.effective_priority, -r.arrival))

    def _preempt(self, rr: RunningRequest, out: Optional[SchedulerOutput] = None) -> None:
        """Free the sequence's KV and queue it again; its cache is recomputed on resume.  In swap mode a fully prefilled
        sequence instead has its blocks copied to host blocks (planned in ``out.swap_out``) and resumes from them."""
        if (out is not None and self.cfg.preemption_mode == "swap" and rr.status is RequestStatus.RUNNING
                and not any(rr is e[0] for e in out.swap_in)):
            # rows worth keeping: every token but the newest, whose row the next decode step writes (a slot this iteration
            # may already have reserved for it is dropped with the rest of the table)
            n_tok = len(rr.all_ids) - 1
            blocks = list(self.cache.table.block_table(rr.id))[: -(-n_tok // self.cfg.block_size)]
            if len(blocks) <= len(self._host_free):
                host = [self._host_free.pop() for _ in blocks]
                rr.swap_host_blocks, rr.swap_tokens = host, n_tok
                out.swap_out.append((rr, blocks, host))
                self.running.remove(rr)
                self.cache.release(rr.id)
                rr.num_preemptions += 1
                self.num_preemptions += 1
                self.num_swaps += 1
                rr.transition(RequestStatus.SWAPPED)
                self.swapped_out.append(rr)
                return
        self.running.remove(rr)
        self.cache.release(rr.id)
        rr.prefill_progress = 0
        rr.cached_prefix = 0
        rr.num_preemptions += 1
        self.num_preemptions += 1
        rr.transition(RequestStatus.PREEMPTED)
        self._push(rr)

    # ------------------------------------------------------------------ planning
    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput()
        self._check_starvation()
        if self.cache.prefix is not None and self.cfg.proactive_evict_above < 1.0:
            self.cache.prefix.proactive_evict(self.cfg.proactive_evict_above)
        budget = self.cfg.max_num_batched_tokens
        # phase 1: every fully prefilled running sequence decodes one token; grow its KV by one slot
        order = sorted(self.running, key=lambda r: (-r.effective_priority, r.arrival))
        for rr in order:
            if rr not in self.running or rr.status is not RequestStatus.RUNNING:
                continue
            if budget <= 0:
                break
            while True:
                try:
                    self.cache.append(rr.id, 1)
                    break
                except OutOfBlocks:
                    victim = self._pick_victim(exclude=(rr,))
                    if victim is None or victim.effective_priority > rr.effective_priority:
                        victim = rr
                    out.preempted.append(victim)
                    if victim in out.decode:
                        out.decode.remove(victim)
                        budget += 1
                    self._preempt(victim, out)
                    if victim is rr:
                        break
            if rr in self.running:
                out.decode.append(rr)
                budget -= 1
        # phase 2: prefill chunks (sequences mid-prefill first, then new admissions)
        prefill_budget = min(budget, self.cfg.max_prefill_tokens)
        for rr in [r for r in self.running if r.status is RequestStatus.PREFILLING]:
            if prefill_budget <= 0:
                break
            n = self._chunk_len(rr, prefill_budget)
            if n > 0:
                out.prefill.append(PrefillChunk(rr, rr.prefill_progress, n))
                prefill_budget -= n
        # swapped sequences come back before anything new is admitted (and hold admissions back while they cannot)
        while self.swapped_out and len(self.running) < self.cfg.max_num_seqs:
            rr = self.swapped_out[0]
            if any(rr is e[0] for e in out.swap_out) or not self.cache.can_admit(rr.swap_tokens + 1):
                break
            try:
                self.cache.table.add_sequence(rr.id, rr.swap_tokens)
            except OutOfBlocks:
                self.cache.table.seqs.pop(rr.id, None)
                break
            self.swapped_out.pop(0)
            out.swap_in.append((rr, rr.swap_host_blocks, list(self.cache.table.block_table(rr.id))))
            self._host_free.extend(rr.swap_host_blocks)
            rr.swap_host_blocks = None
            rr.transition(RequestStatus.RUNNING)
            self.running.append(rr)
        while not self.swapped_out and prefill_budget > 0 and len(self.running) < self.cfg.max_num_seqs:
            rr = self._peek_waiting()
            if rr is None:
                break
            tokens = rr.all_ids[: rr.prefill_target] if rr.output_ids else rr.req.prompt_ids
            if not self.cfg.enable_chunked_prefill and len(tokens) > prefill_budget and out.prefill:
                break
            # room for the whole context plus the first decode slot
            if not self.cache.can_admit(len(tokens) + 1):
                break
            self._pop_waiting(rr)
            try:
                cached = self.cache.admit(rr.id, tokens)
            except OutOfBlocks:
                self._push(rr)
                break
            rr.cached_prefix = cached
            rr.prefill_progress = cached
            rr.transition(RequestStatus.PREFILLING)
            self.running.append(rr)
            n = self._chunk_len(rr, prefill_budget)
            if n > 0:
                out.prefill.append(PrefillChunk(rr, rr.prefill_progress, n))
                prefill_budget -= n
        return out

    def _chunk_len(self, rr: RunningRequest, budget: int) -> int:
        n = min(rr.remaining_prefill, budget)
        if self.cfg.enable_chunked_prefill:
            n = min(n, self.cfg.max_chunk)
        elif n < rr.remaining_prefill:
            return 0
        return n

    # ------------------------------------------------------------------ after the model ran
    def step(self, out: SchedulerOutput, sampled: Dict[str, int]) -> List[RunningRequest]:
        """Account for an executed iteration.  ``sampled`` maps request id -> new token (or, after a speculative step, the
        list of tokens the step produced) for every decode request and for every request whose prefill completed in this
        iteration."""
        finished = []
        for ch in out.prefill:
            rr = ch.request
            rr.prefill_progress += ch.length
            if rr.remaining_prefill == 0 and rr.status is RequestStatus.PREFILLING:
                self.cache.publish(rr.id, rr.req.prompt_ids)
                rr.transition(RequestStatus.RUNNING)
        for rid, tok in sampled.items():
            rr = self.requests[rid]
            if rr.status is not RequestStatus.RUNNING:
                continue
            reason = None
            for t in (tok if isinstance(tok, (list, tuple)) else (tok,)):
                rr.append_token(t)
                reason = rr.should_stop()
                if reason is not None:
                    break
            if reason is None and rr.req.timeout_s is not None and time.monotonic() - rr.arrival > rr.req.timeout_s:
                reason = "timeout"
            if reason is not None:
                rr.finish_reason = reason
                self.running.remove(rr)
                self.cache.release(rr.id)
                rr.transition(RequestStatus.FINISHED)
                self.num_finished += 1
                finished.append(rr)
        return finished

    def stats(self) -> dict:
        return {"waiting": self.num_waiting, "running": len(self.running), "swapped_out": len(self.swapped_out),
                "swaps": self.num_swaps, "preemptions": self.num_preemptions,
                "finished": self.num_finished, "kv": self.cache.stats()}
