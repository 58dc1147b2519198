"""Pipeline parallelism: consecutive layer ranges on consecutive ranks, activations handed over point to point.

Parity: reference ``metal_marlin/distributed/pipeline_parallel.py`` (stage assignment, micro-batch schedule).  Each
stage is a ``Transformer`` holding only its layers (the first stage also the embedding, the last the final norm and
the head); the hand-over is the (hidden, pending delta) pair of the residual stream, moved with non-blocking
``isend`` / ``irecv`` from a side stream so that transfers run under the neighbouring micro-batch's compute.  Prefill and
decode both run micro-batches through the stages back to back (``pipeline_prefill``, ``pipeline_decode_step``).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..models.transformer import BatchMeta, PagedKVStorage, Transformer


def stage_layers(n_layers: int, pp: int) -> List[Tuple[int, int]]:
    """Contiguous, balanced layer ranges (earlier stages take the remainder)."""
    base, rem = divmod(n_layers, pp)
    out, s = [], 0
    for p in range(pp):
        n = base + (1 if p < rem else 0)
        out.append((s, s + n))
        s += n
    return out


class PipelineStage:
    def __init__(self, model: Transformer, stage: int, pp: int, prev_rank: Optional[int], next_rank: Optional[int], group=None):
        self.cfg = model.cfg
        self.stage, self.pp, self.prev, self.next, self.group = stage, pp, prev_rank, next_rank, group
        lo, hi = stage_layers(len(model.layers), pp)[stage]
        self.lo, self.hi = lo, hi
        self.model = model
        self.layers = model.layers[lo:hi]
        self.is_first, self.is_last = stage == 0, stage == pp - 1

    def _run_layers(self, h, d, kv: PagedKVStorage, meta: BatchMeta):
        m = self.model
        for off, L in enumerate(self.layers):
            li = self.lo + off
            h, d = (m._attn_mla if self.cfg.is_mla else m._attn_gqa)(L, li, h, d, kv, meta)
            h, d = (m._mlp_moe if L.router_w is not None else m._mlp_dense)(L, li, h, d)
        return h, d

    # ------------------------------------------------------------------ hand-over
    # Non-blocking point-to-point transfers: the receive of micro-batch i + 1 is posted before micro-batch i is computed and
    # the send of micro-batch i completes while i + 1 is computed.  On CUDA the transfers are issued from a side stream
    # (NCCL runs them on its own stream; events order them against the compute stream), so the copy engines / NVLink work
    # under the layers' kernels instead of between them.
    def _comm_stream(self):
        dev = self.model.device
        if dev.type != "cuda":
            return None
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(dev)
        return self._side

    def post_recv(self, T: int):
        """Start receiving the (hidden, delta) pair of a ``T``-token micro-batch; returns a handle for :meth:`wait_recv`."""
        dev = self.model.device
        buf = torch.empty(2, T, self.cfg.hidden_size, dtype=torch.bfloat16, device=dev)
        side = self._comm_stream()
        if side is None:
            return buf, dist.irecv(buf, src=self.prev, group=self.group), None
        with torch.cuda.stream(side):
            work = dist.irecv(buf, src=self.prev, group=self.group)
            work.wait()                       # orders the side stream after the transfer (the host does not block)
            ev = torch.cuda.Event()
            ev.record(side)
        return buf, work, ev

    def wait_recv(self, handle):
        buf, work, ev = handle
        if ev is None:
            work.wait()
        else:
            torch.cuda.current_stream(self.model.device).wait_event(ev)
            buf.record_stream(torch.cuda.current_stream(self.model.device))
        return buf[0], buf[1]

    def send_async(self, h, d):
        """Start sending; the returned handle keeps the buffer alive until :meth:`wait_send`."""
        buf = torch.stack([h, d if d is not None else torch.zeros_like(h)]).contiguous()
        side = self._comm_stream()
        if side is None:
            return buf, dist.isend(buf, dst=self.next, group=self.group)
        side.wait_stream(torch.cuda.current_stream(self.model.device))      # the pair is complete on the compute stream
        with torch.cuda.stream(side):
            buf.record_stream(side)
            work = dist.isend(buf, dst=self.next, group=self.group)
        return buf, work

    @staticmethod
    def wait_send(handle) -> None:
        handle[1].wait()

    def _recv(self, T: int, device):
        return self.wait_recv(self.post_recv(T))

    def _send(self, h, d):
        self.wait_send(self.send_async(h, d))

    def compute(self, input_ids: torch.Tensor, kv: PagedKVStorage, meta: BatchMeta, rows, recv_handle=None):
        """Layers of this stage on one micro-batch: ``(logits or None, (h, d) to hand over or None)``."""
        if self.is_first:
            h, d = ops.embedding(self.model.embed, input_ids), None
        else:
            h, d = self.wait_recv(recv_handle if recv_handle is not None else self.post_recv(input_ids.numel()))
        h, d = self._run_layers(h, d, kv, meta)
        if self.is_last:
            return self.model.logits(h, d, rows), None
        return None, (h, d)

    def forward(self, input_ids: torch.Tensor, kv: PagedKVStorage, meta: BatchMeta, rows: Optional[torch.Tensor] = None):
        """One micro-batch through this stage, blocking hand-overs.  The last stage returns fp32 logits of ``rows``."""
        out, pair = self.compute(input_ids, kv, meta, rows)
        if pair is not None:
            self._send(*pair)
        return out


def pipeline_prefill(stage: PipelineStage, microbatches: Sequence[Tuple[torch.Tensor, PagedKVStorage, BatchMeta, Optional[torch.Tensor]]],
                     overlap: bool = True, max_inflight_sends: int = 2):
    """Forward-only pipeline schedule (inference has no backward pass, so fill-drain IS the steady-state schedule: stage s
    works on micro-batch i while stage s + 1 works on i - 1).  With ``overlap`` the receive of the next micro-batch is posted
    before the current one is computed and sends complete in the background (at most ``max_inflight_sends`` buffers alive);
    without it every hand-over blocks.  Returns the list of logits on the last stage."""
    outs = []
    if not overlap:
        for ids, kv, meta, rows in microbatches:
            o = stage.forward(ids, kv, meta, rows)
            if o is not None:
                outs.append(o)
        return outs
    sends = []
    nxt = None if stage.is_first or not microbatches else stage.post_recv(microbatches[0][0].numel())
    for i, (ids, kv, meta, rows) in enumerate(microbatches):
        cur = nxt
        nxt = None
        if not stage.is_first and i + 1 < len(microbatches):
            nxt = stage.post_recv(microbatches[i + 1][0].numel())       # arrives while micro-batch i is computed
        o, pair = stage.compute(ids, kv, meta, rows, cur)
        if o is not None:
            outs.append(o)
        if pair is not None:
            sends.append(stage.send_async(*pair))
            while len(sends) > max_inflight_sends:
                stage.wait_send(sends.pop(0))
    for sd in sends:
        stage.wait_send(sd)
    return outs


def pipeline_decode_step(stage: PipelineStage, microbatches: Sequence[Tuple[torch.Tensor, PagedKVStorage, BatchMeta]], overlap: bool = True):
    """One decode step of several independent micro-batches (the running sequences split into up to ``pp`` groups): the groups
    follow each other through the stages, so every stage is busy once the pipe is full instead of idling ``pp - 1`` of ``pp``
    slots as a single decode batch would.  Returns, on the last stage, the logits of every micro-batch in order."""
    return pipeline_prefill(stage, [(ids, kv, meta, None) for ids, kv, meta in microbatches], overlap=overlap)
