"""Direct dispatch of the native extension's operators for the serving loop: a synchronous path for decode (launch on the
current stream, wait), an asynchronous path for prompt work (launch on a side stream, hand back an event handle), and counters.

An operator is named as in the extension's registry (``torch.ops.mmb200.<name>``) or given as a callable; arguments are
the operator's own (tensors and scalars) — launch shapes are chosen inside the kernels' host entry points, so there is no
grid / thread-group argument.  Without the extension or without a GPU, named dispatch is unavailable (``available`` is False
and it raises); callables still run, which is how the bookkeeping is tested on a CPU.

Parity: reference ``serving_cpp/__init__.py`` (``ServingCppDispatcher`` :31 with ``dispatch_sync`` / ``dispatch_async`` / ``wait`` /
``is_complete`` / ``get_metrics`` / ``reset_metrics``; ``ServingCppEngineWrapper`` :201; ``create_serving_cpp_dispatcher`` :299).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Union

import torch


@dataclass
class DispatchHandle:
    index: int
    event: Any = None                    # torch.cuda.Event on a GPU
    result: Any = None
    done: bool = False


class ServingCppDispatcher:
    def __init__(self, device: Optional[Union[str, torch.device]] = None):
        from .. import ops
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self._native = ops.native_available()
        self._available = self._native and self.device.type == "cuda"
        self._side = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self._next = 0
        self.reset_metrics()

    @property
    def available(self) -> bool:
        return self._available

    def _resolve(self, op: Union[str, Callable]) -> Callable:
        if callable(op):
            return op
        if not self._available:
            raise RuntimeError("native serving path not available (the extension is not loaded or there is no GPU)")
        fn = getattr(torch.ops.mmb200, op, None)
        if fn is None:
            raise KeyError(f"the extension has no operator {op!r}")
        return fn

    def dispatch_sync(self, op: Union[str, Callable], *args, **kwargs) -> Any:
        fn = self._resolve(op)
        t0 = time.perf_counter()
        out = fn(*args, **kwargs)
        launched = time.perf_counter()
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        t1 = time.perf_counter()
        self._m["sync_dispatches"] += 1
        self._m["host_launch_s"] += launched - t0
        self._m["sync_wait_s"] += t1 - launched
        return out

    def dispatch_async(self, op: Union[str, Callable], *args, **kwargs) -> DispatchHandle:
        fn = self._resolve(op)
        h = DispatchHandle(self._next)
        self._next += 1
        t0 = time.perf_counter()
        if self._side is not None:
            self._side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._side):
                h.result = fn(*args, **kwargs)
                h.event = torch.cuda.Event()
                h.event.record(self._side)
        else:
            h.result, h.done = fn(*args, **kwargs), True
        self._m["async_dispatches"] += 1
        self._m["host_launch_s"] += time.perf_counter() - t0
        return h

    def wait(self, handle: DispatchHandle) -> Any:
        """Make the current stream (and the host) wait for the work behind ``handle``; returns what the operator returned."""
        if handle.event is not None and not handle.done:
            torch.cuda.current_stream(self.device).wait_event(handle.event)
            handle.event.synchronize()
        handle.done = True
        self._m["waits"] += 1
        return handle.result

    def is_complete(self, handle: DispatchHandle) -> bool:
        if handle.done:
            return True
        if handle.event is not None and handle.event.query():
            handle.done = True
        return handle.done

    def get_metrics(self) -> Dict[str, Any]:
        m = dict(self._m)
        n = m["sync_dispatches"] + m["async_dispatches"]
        m["total_dispatches"] = n
        m["avg_host_launch_us"] = 1e6 * m["host_launch_s"] / n if n else 0.0
        m["available"] = self._available
        return m

    def reset_metrics(self) -> None:
        self._m = {"sync_dispatches": 0, "async_dispatches": 0, "waits": 0, "host_launch_s": 0.0, "sync_wait_s": 0.0}


class ServingCppEngineWrapper:
    """The two dispatch modes under the names the serving loop uses: decode work waits, prompt work overlaps."""

    def __init__(self, engine: Any = None, dispatcher: Optional[ServingCppDispatcher] = None):
        self.engine = engine
        self.dispatcher = dispatcher or ServingCppDispatcher()
        self.decode_calls = self.prefill_calls = 0

    @property
    def available(self) -> bool:
        return self.dispatcher.available

    def dispatch_for_decode(self, op: Union[str, Callable], *args, **kwargs) -> Any:
        self.decode_calls += 1
        return self.dispatcher.dispatch_sync(op, *args, **kwargs)

    def dispatch_for_prefill(self, op: Union[str, Callable], *args, **kwargs) -> DispatchHandle:
        self.prefill_calls += 1
        return self.dispatcher.dispatch_async(op, *args, **kwargs)

    def wait(self, handle: DispatchHandle) -> Any:
        return self.dispatcher.wait(handle)

    def get_metrics(self) -> Dict[str, Any]:
        return {**self.dispatcher.get_metrics(), "decode_calls": self.decode_calls, "prefill_calls": self.prefill_calls}


def create_serving_cpp_dispatcher(device=None) -> Optional[ServingCppDispatcher]:
    """A dispatcher when the native path is available, else None."""
    d = ServingCppDispatcher(device)
    return d if d.available else None
