"""First-come-first-served scheduler: arrival-ordered waiting queue, a swapped queue that is re-admitted first, prefill
strategies (arrival order / shortest prompt first / longest prompt first), batch insertion policies (enqueue / merge at the
front / drop when the queue is full) with insertion statistics, victim selection by generated-token count, and per-request
prefix-cache accounting.  It plans iterations through the same budget / chunking / paged-cache machinery as the
continuous-batching scheduler (``engine/scheduler.py``), so the engine loop can run either one
(``EngineConfig.scheduler_policy = "fcfs"``).

Parity: reference ``metal_marlin/serving/scheduler.py``: ``PrefillStrategy`` ``:308``, ``SchedulerConfig`` ``:317``,
``FCFSScheduler`` ``:329`` (``schedule`` ``:411``: running sequences first, then swapped ones, then waiting ones in strategy
order; ``_select_preempt_victim`` ``:658``: most generated tokens; ``get_cache_info`` ``:740``), ``InsertionPolicy`` ``:769``,
``QueueFullError`` ``:777``, ``BatchScheduler`` ``:783`` (``insert_batch`` ``:870``, ``insert_batch_front`` ``:928``,
``add_request_front`` ``:943``, ``insertion_stats`` ``:972``, ``queue_utilization`` ``:994``, ``clear_waiting`` ``:1006``).
"""
from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass
from typing import Deque, Dict, Iterable, List, Optional

from ..kv.paged import PagedKVCache
from .request import GenerationRequest, RequestStatus, RunningRequest
from .scheduler import BatchScheduler, PreemptionPolicy, QueueFullError, SchedulerConfig


class PrefillStrategy(enum.Enum):
    FCFS = "fcfs"                          # arrival order
    SHORTEST_FIRST = "shortest_first"      # shorter prompts first: lower time to first token
    LONGEST_FIRST = "longest_first"        # longer prompts first: fuller prefill batches


class InsertionPolicy(enum.Enum):
    ENQUEUE = "enqueue"                    # back of the waiting queue, order kept
    MERGE = "merge"                        # front of the waiting queue, order kept
    DROP_IF_FULL = "drop_if_full"          # the whole batch is dropped unless all of it fits


@dataclass
class CacheInfo:
    """How much of a request's prompt the prefix cache served at admission."""
    cached_blocks: int = 0
    cached_tokens: int = 0
    uncached_tokens: int = 0

    @property
    def cache_hit(self) -> bool:
        return self.cached_tokens > 0

    @property
    def total_tokens(self) -> int:
        return self.cached_tokens + self.uncached_tokens


class FCFSScheduler(BatchScheduler):
    def __init__(self, config: SchedulerConfig, cache: PagedKVCache, *, prefill_strategy: PrefillStrategy = PrefillStrategy.FCFS,
                 max_queue_size: Optional[int] = None):
        config.fcfs = True
        if config.preemption_policy is PreemptionPolicy.LOWEST_PRIORITY:
            config.preemption_policy = PreemptionPolicy.MOST_TOKENS      # priorities do not exist here
        if max_queue_size is not None:
            config.max_waiting = max_queue_size
        super().__init__(config, cache)
        self.prefill_strategy = PrefillStrategy(prefill_strategy)
        self.waiting: Deque[RunningRequest] = deque()
        self.swapped: Deque[RunningRequest] = deque()
        self._ins = {"total_inserted": 0, "total_dropped": 0, "batch_insertions": 0}

    # ------------------------------------------------------------------ queues
    @property
    def max_queue_size(self) -> int:
        return self.cfg.max_waiting

    @property
    def num_waiting(self) -> int:
        return len(self.waiting)

    @property
    def num_swapped(self) -> int:
        return len(self.swapped)

    @property
    def num_running(self) -> int:
        return len(self.running)

    def has_work(self) -> bool:
        return bool(self.waiting or self.swapped or self.running or self.swapped_out)

    has_pending_work = property(has_work)

    def _push(self, rr: RunningRequest) -> None:
        # a preempted sequence waits in the swapped queue and is re-admitted before anything new
        (self.swapped if rr.status is RequestStatus.PREEMPTED else self.waiting).append(rr)

    def _strategy_order(self) -> List[RunningRequest]:
        w = list(self.waiting)
        if self.prefill_strategy is PrefillStrategy.SHORTEST_FIRST:
            return sorted(w, key=lambda r: len(r.req.prompt_ids))          # stable: ties keep arrival order
        if self.prefill_strategy is PrefillStrategy.LONGEST_FIRST:
            return sorted(w, key=lambda r: -len(r.req.prompt_ids))
        return w

    def _peek_waiting(self) -> Optional[RunningRequest]:
        if self.swapped:
            return self.swapped[0]
        if not self.waiting:
            return None
        if self.prefill_strategy is PrefillStrategy.FCFS:
            return self.waiting[0]
        return self._strategy_order()[0]

    def _pop_waiting(self, rr: RunningRequest) -> None:
        if self.swapped and self.swapped[0] is rr:
            self.swapped.popleft()
        else:
            self.waiting.remove(rr)

    def _drop_waiting(self, rr: RunningRequest) -> None:
        for q in (self.waiting, self.swapped):
            if rr in q:
                q.remove(rr)

    def _check_starvation(self) -> None:
        return

    # ------------------------------------------------------------------ insertion
    def _room(self) -> int:
        return max(0, self.cfg.max_waiting - len(self.waiting))

    def _new(self, req: GenerationRequest) -> RunningRequest:
        if len(req.prompt_ids) + req.max_new_tokens > self.cfg.max_model_len:
            raise ValueError("context_length_exceeded")
        rr = RunningRequest(req)
        self.requests[rr.id] = rr
        return rr

    def add_request(self, req: GenerationRequest) -> RunningRequest:
        if self._room() == 0:
            raise QueueFullError(f"cannot add {req.request_id}: waiting queue is full ({len(self.waiting)} >= {self.cfg.max_waiting})")
        rr = self._new(req)
        self.waiting.append(rr)
        self._ins["total_inserted"] += 1
        return rr

    def add_request_front(self, req: GenerationRequest) -> RunningRequest:
        """Queue one request ahead of everything that is waiting."""
        if self._room() == 0:
            raise QueueFullError(f"cannot add {req.request_id}: waiting queue is full ({len(self.waiting)} >= {self.cfg.max_waiting})")
        rr = self._new(req)
        self.waiting.appendleft(rr)
        self._ins["total_inserted"] += 1
        return rr

    def insert_batch(self, requests: Iterable[GenerationRequest], policy: InsertionPolicy = InsertionPolicy.ENQUEUE) -> int:
        """Insert several requests at once; returns how many were queued.  ``ENQUEUE`` and ``MERGE`` queue as many as fit (in
        order) and count the rest as dropped; ``DROP_IF_FULL`` queues all of them or none."""
        reqs = list(requests)
        policy = InsertionPolicy(policy)
        self._ins["batch_insertions"] += 1
        room = self._room()
        if policy is InsertionPolicy.DROP_IF_FULL and len(reqs) > room:
            self._ins["total_dropped"] += len(reqs)
            return 0
        take, rest = reqs[:room], reqs[room:]
        rrs = [self._new(r) for r in take]
        if policy is InsertionPolicy.MERGE:
            self.waiting.extendleft(reversed(rrs))
        else:
            self.waiting.extend(rrs)
        self._ins["total_inserted"] += len(rrs)
        self._ins["total_dropped"] += len(rest)
        return len(rrs)

    def insert_batch_front(self, requests: Iterable[GenerationRequest]) -> int:
        return self.insert_batch(requests, InsertionPolicy.MERGE)

    def insertion_stats(self) -> Dict[str, int]:
        return dict(self._ins)

    def reset_insertion_stats(self) -> None:
        for k in self._ins:
            self._ins[k] = 0

    def queue_utilization(self) -> float:
        return len(self.waiting) / self.cfg.max_waiting if self.cfg.max_waiting > 0 else 0.0

    def clear_waiting(self) -> int:
        """Abort everything that has not started; returns the number of requests removed."""
        n = 0
        for rr in list(self.waiting):
            n += int(self.abort(rr.id))
        return n

    # ------------------------------------------------------------------ accounting
    def get_cache_info(self, request_id: str) -> Optional[CacheInfo]:
        rr = self.requests.get(request_id)
        if rr is None or rr.status is RequestStatus.WAITING:
            return None
        bs = self.cfg.block_size
        total = len(rr.req.prompt_ids)
        return CacheInfo(cached_blocks=rr.cached_prefix // bs, cached_tokens=rr.cached_prefix, uncached_tokens=max(0, total - rr.cached_prefix))

    def free_finished(self) -> List[RunningRequest]:
        """Drop the bookkeeping of finished / aborted / failed requests (their cache blocks were released when they ended)."""
        done = [rr for rr in self.requests.values() if rr.status in (RequestStatus.FINISHED, RequestStatus.ABORTED, RequestStatus.FAILED)]
        for rr in done:
            del self.requests[rr.id]
        return done

    def stats(self) -> dict:
        s = super().stats()
        s.update(swapped=len(self.swapped), prefill_strategy=self.prefill_strategy.value, queue_utilization=round(self.queue_utilization(), 4),
                 **{f"insert_{k}": v for k, v in self._ins.items()})
        return s
