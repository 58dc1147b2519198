"""Request model of the serving engine: generation request, status FSM, scheduler output.

Parity: reference ``metal_marlin/serving/request.py:52-431`` (``GenerationRequest``,
``RequestStatus``, ``RunningRequest`` with legal transitions, ``SchedulerOutput``) and
``metal_marlin/serving/continuous_batch.py:54-180`` (``RequestPriority``, ``RequestState``).
"""
from __future__ import annotations

import enum
import itertools
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from .session import SamplingParams


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    PREFILLING = "prefilling"
    RUNNING = "running"
    PREEMPTED = "preempted"
    SWAPPED = "swapped"          # preempted with its cache rows parked in host memory (resumes without recomputing)
    FINISHED = "finished"
    ABORTED = "aborted"
    FAILED = "failed"


_LEGAL = {
    RequestStatus.WAITING: {RequestStatus.PREFILLING, RequestStatus.ABORTED, RequestStatus.FAILED},
    RequestStatus.PREFILLING: {RequestStatus.RUNNING, RequestStatus.PREEMPTED, RequestStatus.FINISHED,
                               RequestStatus.ABORTED, RequestStatus.FAILED},
    RequestStatus.RUNNING: {RequestStatus.FINISHED, RequestStatus.PREEMPTED, RequestStatus.SWAPPED, RequestStatus.ABORTED,
                            RequestStatus.FAILED},
    RequestStatus.SWAPPED: {RequestStatus.RUNNING, RequestStatus.ABORTED, RequestStatus.FAILED},
    RequestStatus.PREEMPTED: {RequestStatus.PREFILLING, RequestStatus.WAITING, RequestStatus.ABORTED, RequestStatus.FAILED},
    RequestStatus.FINISHED: set(), RequestStatus.ABORTED: set(), RequestStatus.FAILED: set(),
}


class RequestPriority(enum.IntEnum):
    LOW = 0
    NORMAL = 1
    HIGH = 2
    REALTIME = 3


class IllegalTransition(RuntimeError):
    pass


_ids = itertools.count()


@dataclass
class GenerationRequest:
    prompt_ids: List[int]
    max_new_tokens: int = 16
    sampling: SamplingParams = field(default_factory=SamplingParams)
    eos_ids: Sequence[int] = ()
    stop_token_ids: Sequence[int] = ()
    priority: RequestPriority = RequestPriority.NORMAL
    request_id: str = ""
    timeout_s: Optional[float] = None
    on_token: Optional[Callable[[str, int], None]] = None     # streaming callback (request_id, token)

    def __post_init__(self):
        if not self.request_id:
            self.request_id = f"req-{next(_ids)}"
        if not self.prompt_ids:
            raise ValueError("empty prompt")


@dataclass
class RunningRequest:
    """Mutable per-request state owned by the scheduler / engine thread."""
    req: GenerationRequest
    status: RequestStatus = RequestStatus.WAITING
    output_ids: List[int] = field(default_factory=list)
    prefill_progress: int = 0            # prompt(+regenerated) tokens whose KV is in the cache
    cached_prefix: int = 0               # tokens served by the prefix cache at admission
    arrival: float = field(default_factory=time.monotonic)
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    finish_reason: Optional[str] = None
    num_preemptions: int = 0
    effective_priority: int = 0
    error: Optional[str] = None
    done: threading.Event = field(default_factory=threading.Event)
    spec_accepted: int = 0
    spec_proposed: int = 0
    swap_host_blocks: Optional[List[int]] = None     # host blocks holding the cache rows while the request is SWAPPED
    swap_tokens: int = 0                             # rows those blocks hold

    def __post_init__(self):
        self.effective_priority = int(self.req.priority)

    @property
    def id(self) -> str:
        return self.req.request_id

    @property
    def all_ids(self) -> List[int]:
        return self.req.prompt_ids + self.output_ids

    @property
    def prefill_target(self) -> int:
        """Tokens that must be in the cache before the next decode step: the prompt plus, after a
        preemption, all generated tokens but the last (which is the next decode input)."""
        return len(self.req.prompt_ids) + max(0, len(self.output_ids) - 1)

    @property
    def remaining_prefill(self) -> int:
        return max(0, self.prefill_target - self.prefill_progress)

    def transition(self, new: RequestStatus) -> None:
        if new not in _LEGAL[self.status]:
            raise IllegalTransition(f"{self.status.value} -> {new.value}")
        self.status = new
        if new in (RequestStatus.FINISHED, RequestStatus.ABORTED, RequestStatus.FAILED):
            self.finish_time = time.monotonic()
            self.done.set()

    def append_token(self, tok: int) -> None:
        if self.first_token_time is None:
            self.first_token_time = time.monotonic()
        self.output_ids.append(int(tok))
        if self.req.on_token is not None:
            self.req.on_token(self.id, int(tok))

    def should_stop(self) -> Optional[str]:
        if self.output_ids and (self.output_ids[-1] in self.req.eos_ids or self.output_ids[-1] in self.req.stop_token_ids):
            return "stop"
        if len(self.output_ids) >= self.req.max_new_tokens:
            return "length"
        return None

    # latency metrics (seconds)
    @property
    def ttft(self) -> Optional[float]:
        return None if self.first_token_time is None else self.first_token_time - self.arrival

    @property
    def latency(self) -> Optional[float]:
        return None if self.finish_time is None else self.finish_time - self.arrival


@dataclass
class PrefillChunk:
    request: RunningRequest
    start: int
    length: int


@dataclass
class SchedulerOutput:
    prefill: List[PrefillChunk] = field(default_factory=list)
    decode: List[RunningRequest] = field(default_factory=list)
    preempted: List[RunningRequest] = field(default_factory=list)
    # cache blocks to move before the model runs, in this order: (request, device blocks, host blocks) out, then
    # (request, host blocks, device blocks) in
    swap_out: List[tuple] = field(default_factory=list)
    swap_in: List[tuple] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(c.length for c in self.prefill) + len(self.decode)

    @property
    def is_empty(self) -> bool:
        return not self.prefill and not self.decode
